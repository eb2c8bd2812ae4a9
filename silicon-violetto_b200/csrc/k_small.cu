// The step's small kernels: embedding, K/V write with RoPE, the scalar attention used as a
// cross-check, the split merge, row preparation, and the integer tail (sample, accept,
// kv_compact, replay_draft).
#include <cfloat>

#include "kernels.h"
#include "sampling.cuh"

namespace vlt {

// ---------------------------------------------------------------- embedding
// kernels.metal:82-114 `embed`, for a plain decoder (the embedding is not normed). Resolves a
// GPU-fed token in place: its id from feed[slot], its position from its node's depth, the rows
// it sees from the node. meta[t] = (slot, lens[slot] + depth). One block per token.
__global__ void embed_kernel(const uint16_t* __restrict__ table, uint32_t* tokens, float* __restrict__ out, const uint32_t* __restrict__ tin,
                             uint32_t* meta, const uint32_t* __restrict__ lens, const uint32_t* __restrict__ feed, const uint32_t* __restrict__ tree,
                             uint32_t* vis, uint32_t d, uint32_t vocab) {
    pdl_start();
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const uint32_t slot = tin[2 * t];
    uint32_t tok = tokens[t], depth = tin[2 * t + 1];
    const bool fed = tok >= FEED_ROW;
    uint32_t node = 0;
    if (fed) {
        const uint32_t i = tok - FEED_ROW;
        node = tree[slot * FEED_W + i];
        tok = feed[slot * FEED_W + i];
        depth = node_depth(node);
    }
    // An id past the vocabulary can only come from the device (a row of NaN logits has no argmax): read it as 0
    // rather than index out of the table.
    if (tok >= vocab) tok = 0;
    const uint32_t* row = reinterpret_cast<const uint32_t*>(table + size_t(tok) * d);
    float2* o = reinterpret_cast<float2*>(out + size_t(t) * d);
    for (uint32_t i = tid; i < d / 2; i += blockDim.x) {
        const uint32_t w = row[i];
        o[i] = make_float2(bf16lo(w), bf16hi(w));
    }
    __syncthreads();  // every thread has read tokens[t]
    if (tid == 0) {
        if (fed) vis[t] = node_sees(node);
        tokens[t] = tok;
        meta[2 * t] = slot;
        meta[2 * t + 1] = lens[slot] + depth;
    }
}

void launch_embed(const uint16_t* table, uint32_t* tokens, float* out, const uint32_t* tin, uint32_t* meta, const uint32_t* lens,
                  const uint32_t* feed, const uint32_t* tree, uint32_t* vis, uint32_t n, uint32_t d, uint32_t vocab, cudaStream_t s) {
    launch_pdl(embed_kernel, n, 128, 0, s, table, tokens, out, tin, meta, lens, feed, tree, vis, d, vocab);
}

// ------------------------------------------------------- K/V into the cache
// kernels.metal:749-801 `qkv_post`, a plain decoder's part of it: RoPE on k (interleaved
// pairs, kernels.metal:727-736, angle of the token's position), k and v rounded to bf16 and
// written at the token's cache row (its run's first position + its row, kernels.metal:74-77).
// One block per token, one warp per kv head, a lane per pair of dims (head_dim 64). The same
// warps then leave q as the tensor-core attention wants it: RoPE, the softmax scale * log2(e)
// folded in, rounded to bf16 (kernels.metal:776-789 does this for q in the same kernel).
__global__ void qkv_post_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin,
                                const float* __restrict__ rope, uint16_t* k_cache, uint16_t* v_cache, const uint32_t* __restrict__ page_table,
                                KvArgs kv, uint32_t layer, uint32_t n_heads, float scale_log2, uint32_t* __restrict__ q_b, const uint32_t* __restrict__ cpos_in) {
    pdl_start();
    const uint32_t t = blockIdx.x, g = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], row = tin[2 * t + 1];
    const uint32_t cpos = cpos_in ? cpos_in[t] : meta[2 * (t - row) + 1] + row;
    const uint32_t qw = (n_heads + 2 * kv.n_kv) * kv.hd;
    const float* kp = qkv + size_t(t) * qw + size_t(n_heads) * kv.hd + g * kv.hd;
    const float* vp = kp + size_t(kv.n_kv) * kv.hd;
    const float2 cs = reinterpret_cast<const float2*>(rope)[size_t(pos) * (kv.hd / 2) + lane];
    const float2 k = reinterpret_cast<const float2*>(kp)[lane];
    const float2 v = reinterpret_cast<const float2*>(vp)[lane];
    const float r0 = __fadd_rn(__fmul_rn(cs.x, k.x), __fmul_rn(cs.y, k.y));
    const float r1 = __fsub_rn(__fmul_rn(cs.x, k.y), __fmul_rn(cs.y, k.x));
    if (cpos != NO_TOK) {  // (the drafter's passes leave out the rows that are not on the accepted path)
        const size_t at = kv_row(kv, layer, page_table, slot, g, cpos);
        reinterpret_cast<uint32_t*>(k_cache + at)[lane] = pack_bf16(r0, r1);
        reinterpret_cast<uint32_t*>(v_cache + at)[lane] = pack_bf16(v.x, v.y);
    }
    if (q_b) {
        for (uint32_t h = g; h < n_heads; h += kv.n_kv) {
            const float2 q = reinterpret_cast<const float2*>(qkv + size_t(t) * qw + h * kv.hd)[lane];
            const float q0 = __fadd_rn(__fmul_rn(cs.x, q.x), __fmul_rn(cs.y, q.y));
            const float q1 = __fsub_rn(__fmul_rn(cs.x, q.y), __fmul_rn(cs.y, q.x));
            q_b[(size_t(t) * n_heads + h) * (kv.hd / 2) + lane] = pack_bf16(__fmul_rn(q0, scale_log2), __fmul_rn(q1, scale_log2));
        }
    }
}

void launch_qkv_post(const float* qkv, const uint32_t* meta, const uint32_t* tin, const float* rope, uint16_t* k_cache, uint16_t* v_cache,
                     const uint32_t* page_table, KvArgs kv, uint32_t layer, uint32_t n, uint32_t n_heads, float scale_log2, uint16_t* q_b, const uint32_t* cpos, cudaStream_t s) {
    launch_pdl(qkv_post_kernel, n, 32 * kv.n_kv, 0, s, qkv, meta, tin, rope, k_cache, v_cache, page_table, kv, layer, n_heads, scale_log2, reinterpret_cast<uint32_t*>(q_b), cpos);
}

// q | k | v of every token with RoPE applied to the q and k heads, in fp32 and unscaled: what engine.rs:183's `qkv`
// capture holds ("after the norms, RoPE and value embeddings"). One block per token, a thread per pair of dims.
__global__ void qkv_capture_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const float* __restrict__ rope, uint32_t n_heads, KvArgs kv,
                                   float* out) {
    const uint32_t t = blockIdx.x, pos = meta[2 * t + 1], half = kv.hd / 2, qw = (n_heads + 2 * kv.n_kv) * kv.hd;
    for (uint32_t i = threadIdx.x; i < qw / 2; i += blockDim.x) {
        const uint32_t head = i / half, pr = i % half;
        const float2 x = reinterpret_cast<const float2*>(qkv + size_t(t) * qw)[i];
        float2 y = x;
        if (head < n_heads + kv.n_kv) {
            const float2 cs = reinterpret_cast<const float2*>(rope)[size_t(pos) * half + pr];
            y.x = __fadd_rn(__fmul_rn(cs.x, x.x), __fmul_rn(cs.y, x.y));
            y.y = __fsub_rn(__fmul_rn(cs.x, x.y), __fmul_rn(cs.y, x.x));
        }
        reinterpret_cast<float2*>(out + size_t(t) * qw)[i] = y;
    }
}
void launch_qkv_capture(const float* qkv, const uint32_t* meta, const float* rope, uint32_t n, uint32_t n_heads, KvArgs kv, float* out, cudaStream_t s) {
    if (!n) return;
    qkv_capture_kernel<<<n, 256, 0, s>>>(qkv, meta, rope, n_heads, kv, out);
    launch_counter()++;
}

// ----------------------------------------------- scalar attention (cross-check)
// One block of 128 threads per (token, head): every thread takes keys tid, tid + 128, ... of the
// token's visible keys -- the cache below its tile's first position, then the tile's rows its
// `vis` mask names (kernels.metal:989-990) -- with an online softmax, and the block merges.
__global__ void attn_plain_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tiles,
                                  const uint32_t* __restrict__ vis, const float* __restrict__ rope, const uint16_t* __restrict__ k_cache,
                                  const uint16_t* __restrict__ v_cache, const uint32_t* __restrict__ page_table, KvArgs kv, uint32_t layer,
                                  uint32_t n_heads, float scale_log2, float* out) {
    constexpr uint32_t HD = 64, NT = 128;
    __shared__ float q[HD];
    __shared__ float red_m[NT], red_l[NT];
    __shared__ float red_o[NT][HD + 1];
    const uint32_t tile = blockIdx.x, i = blockIdx.y, h = blockIdx.z, tid = threadIdx.x;
    const uint32_t t0 = tiles[2 * tile], T = tiles[2 * tile + 1];
    if (i >= T) return;
    const uint32_t t = t0 + i, g = h / (n_heads / kv.n_kv);
    const uint32_t slot = meta[2 * t0], p0 = meta[2 * t0 + 1], pos = meta[2 * t + 1], mask = vis[t];
    const uint32_t qw = (n_heads + 2 * kv.n_kv) * HD;
    if (tid < HD / 2) {
        const float2 v = reinterpret_cast<const float2*>(qkv + size_t(t) * qw + h * HD)[tid];
        const float2 cs = reinterpret_cast<const float2*>(rope)[size_t(pos) * (HD / 2) + tid];
        const float r0 = __fadd_rn(__fmul_rn(cs.x, v.x), __fmul_rn(cs.y, v.y));
        const float r1 = __fsub_rn(__fmul_rn(cs.x, v.y), __fmul_rn(cs.y, v.x));
        q[2 * tid] = round_bf16(__fmul_rn(r0, scale_log2));
        q[2 * tid + 1] = round_bf16(__fmul_rn(r1, scale_log2));
    }
    __syncthreads();
    float m = -INFINITY, l = 0.0f, o[HD];
#pragma unroll
    for (uint32_t d = 0; d < HD; d++) o[d] = 0.0f;
    for (uint32_t kp = tid; kp < p0 + T; kp += NT) {
        if (kp >= p0 && !((mask >> (kp - p0)) & 1u)) continue;
        const size_t at = kv_row(kv, layer, page_table, slot, g, kp);
        const uint4* kr = reinterpret_cast<const uint4*>(k_cache + at);
        float sc = 0.0f;
#pragma unroll
        for (uint32_t c = 0; c < HD / 8; c++) {
            const uint4 w = kr[c];
            sc += q[8 * c] * bf16lo(w.x) + q[8 * c + 1] * bf16hi(w.x) + q[8 * c + 2] * bf16lo(w.y) + q[8 * c + 3] * bf16hi(w.y) +
                  q[8 * c + 4] * bf16lo(w.z) + q[8 * c + 5] * bf16hi(w.z) + q[8 * c + 6] * bf16lo(w.w) + q[8 * c + 7] * bf16hi(w.w);
        }
        const float mn = fmaxf(m, sc), corr = exp2f(m - mn), p = exp2f(sc - mn);
        l = l * corr + p;
        const uint4* vr = reinterpret_cast<const uint4*>(v_cache + at);
#pragma unroll
        for (uint32_t c = 0; c < HD / 8; c++) {
            const uint4 w = vr[c];
            o[8 * c] = o[8 * c] * corr + p * bf16lo(w.x);
            o[8 * c + 1] = o[8 * c + 1] * corr + p * bf16hi(w.x);
            o[8 * c + 2] = o[8 * c + 2] * corr + p * bf16lo(w.y);
            o[8 * c + 3] = o[8 * c + 3] * corr + p * bf16hi(w.y);
            o[8 * c + 4] = o[8 * c + 4] * corr + p * bf16lo(w.z);
            o[8 * c + 5] = o[8 * c + 5] * corr + p * bf16hi(w.z);
            o[8 * c + 6] = o[8 * c + 6] * corr + p * bf16lo(w.w);
            o[8 * c + 7] = o[8 * c + 7] * corr + p * bf16hi(w.w);
        }
        m = mn;
    }
    red_m[tid] = m;
    red_l[tid] = l;
#pragma unroll
    for (uint32_t d = 0; d < HD; d++) red_o[tid][d] = o[d];
    __syncthreads();
    if (tid < HD) {
        float mm = -INFINITY;
        for (uint32_t j = 0; j < NT; j++) mm = fmaxf(mm, red_m[j]);
        float ll = 0.0f, oo = 0.0f;
        for (uint32_t j = 0; j < NT; j++) {
            if (red_m[j] == -INFINITY) continue;
            const float w = exp2f(red_m[j] - mm);
            ll += red_l[j] * w;
            oo += red_o[j][tid] * w;
        }
        out[size_t(t) * n_heads * HD + h * HD + tid] = oo / ll;
    }
}

void launch_attn_plain(const float* qkv, const uint32_t* meta, const uint32_t* tiles, const uint32_t* vis, const float* rope, const uint16_t* k_cache,
                       const uint16_t* v_cache, const uint32_t* page_table, KvArgs kv, uint32_t layer, uint32_t n_tiles, uint32_t n_heads,
                       float scale_log2, float* out, cudaStream_t s) {
    attn_plain_kernel<<<dim3(n_tiles, VERIFY_T, n_heads), 128, 0, s>>>(qkv, meta, tiles, vis, rope, k_cache, v_cache, page_table, kv, layer, n_heads,
                                                                      scale_log2, out);
    launch_counter()++;
}

// ------------------------------------------------------------ split merge
// kernels.metal:1314-1362 `attn_dec_reduce`, with a running maximum: the partials of a
// (token, head) are (m, l, o[64]) per key split; out = sum(o_s 2^(m_s - M)) / sum(l_s 2^(m_s - M)).
// One block per token and four heads, 64 threads a head.
// Splits past a tile's keys hold m = -inf (the attention kernel writes every slot).
// COMBINE_HEADS heads per block, 64 threads each: four when there are blocks enough to fill the GPU anyway (fewer,
// fatter blocks schedule faster), one otherwise.
template <uint32_t COMBINE_HEADS>
__global__ void __launch_bounds__(64 * COMBINE_HEADS) attn_combine_kernel(const float* __restrict__ part, uint32_t max_splits, uint32_t n_heads, float* out,
                                                                          uint16_t* out_b) {
    pdl_start();
    __shared__ float ws[COMBINE_HEADS][64];   // the splits' weights 2^(m_s - M), 0 for an empty split
    __shared__ float lws[COMBINE_HEADS][64];  // l_s times that
    __shared__ float red[COMBINE_HEADS][2];
    const uint32_t t = blockIdx.x, hl = threadIdx.x / 64, h = blockIdx.y * COMBINE_HEADS + hl, d = threadIdx.x % 64;
    const bool live = h < n_heads;
    const float* pp = part + (size_t(t) * n_heads + (live ? h : 0)) * max_splits * ATTN_PART;
    // A thread per split for the statistics (at most 64 splits, engine.cu `attention_split`), then a thread
    // per dim with the splits' loads independent of each other.
    // The first eight splits' values are asked for together with the statistics (they do not depend on them): one
    // round trip to L2 instead of two.
    float v8[8];
#pragma unroll
    for (uint32_t s = 0; s < 8; s++) v8[s] = s < max_splits ? pp[s * ATTN_PART + 4 + d] : 0.0f;
    const bool has = d < max_splits;
    const float ms = has ? pp[d * ATTN_PART] : -INFINITY;
    const float ls = has ? pp[d * ATTN_PART + 1] : 0.0f;
    float mm = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    if (d % 32 == 0) red[hl][d / 32] = mm;
    __syncthreads();
    mm = fmaxf(red[hl][0], red[hl][1]);
    const float w = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
    ws[hl][d] = w;
    lws[hl][d] = ls * w;  // summed in split order below, so that the result does not depend on the warp layout
    __syncthreads();
    float ll = 0.0f, oo = 0.0f;
    for (uint32_t s = 0; s < max_splits; s++) ll += lws[hl][s];
#pragma unroll
    for (uint32_t s = 0; s < 8; s++)  // an empty split's o was never written: whatever is there must not count
        if (s < max_splits) oo += ws[hl][s] == 0.0f ? 0.0f : v8[s] * ws[hl][s];
#pragma unroll 8
    for (uint32_t s = 8; s < max_splits; s++) {
        const float v = pp[s * ATTN_PART + 4 + d];
        oo += ws[hl][s] == 0.0f ? 0.0f : v * ws[hl][s];
    }
    if (!live) return;
    const float r = oo / ll;
    const size_t at = size_t(t) * n_heads * 64 + h * 64 + d;
    out[at] = r;
    if (out_b) out_b[at] = f32_to_bf16(r);
}

// The same merge for many splits (a long context read by few streams): one block per (token, head), four groups of 64
// threads that take every fourth split each, so that a thread has at most 16 loads and all of them in flight at once;
// the groups' sums are added in group order.
__global__ void __launch_bounds__(256) attn_combine_wide_kernel(const float* __restrict__ part, uint32_t max_splits, uint32_t n_heads, float* out, uint16_t* out_b) {
    pdl_start();
    __shared__ float ws[64], lws[64], red[8], og[4][64];
    const uint32_t t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, grp = tid / 64, d = tid % 64;
    const float* pp = part + (size_t(t) * n_heads + h) * max_splits * ATTN_PART;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {  // (asked for first: they do not depend on the statistics)
        const uint32_t s = grp + 4 * i;
        v[i] = s < max_splits ? pp[s * ATTN_PART + 4 + d] : 0.0f;
    }
    const bool has = tid < max_splits;  // at most 64 splits (engine.cu `attention_split`)
    const float ms = has ? pp[tid * ATTN_PART] : -INFINITY;
    const float ls = has ? pp[tid * ATTN_PART + 1] : 0.0f;
    float mm = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    if (tid % 32 == 0) red[tid / 32] = mm;
    __syncthreads();
    mm = fmaxf(red[0], red[1]);
    if (tid < 64) {
        const float w = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
        ws[tid] = w;
        lws[tid] = ls * w;
    }
    __syncthreads();
    float oo = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t s = grp + 4 * i;
        if (s < max_splits && ws[s] != 0.0f) oo += v[i] * ws[s];  // an empty split's o was never written: whatever is there must not count
    }
    og[grp][d] = oo;
    __syncthreads();
    if (tid >= 64) return;
    float ll = 0.0f;
    for (uint32_t s = 0; s < max_splits; s++) ll += lws[s];
    const float r = (((og[0][d] + og[1][d]) + og[2][d]) + og[3][d]) / ll;
    const size_t at = size_t(t) * n_heads * 64 + h * 64 + d;
    out[at] = r;
    if (out_b) out_b[at] = f32_to_bf16(r);
}

void launch_attn_combine(const AttnArgs& a, cudaStream_t s) {
    if (a.max_splits > 8) launch_pdl(attn_combine_wide_kernel, dim3(a.n, a.n_heads), 256, 0, s, a.part, a.max_splits, a.n_heads, a.out, a.out_b);
    else if (a.n * a.n_heads >= 2048) launch_pdl(attn_combine_kernel<4>, dim3(a.n, (a.n_heads + 3) / 4), 256, 0, s, a.part, a.max_splits, a.n_heads, a.out, a.out_b);
    else launch_pdl(attn_combine_kernel<1>, dim3(a.n, a.n_heads), 64, 0, s, a.part, a.max_splits, a.n_heads, a.out, a.out_b);
}

// ------------------------------------------------------------- row preparation
// kernels.metal:117-148 `rmsnorm_rows` / `tap_rows`: out[r] = in[rows[r]] (optionally normed,
// optionally rounded to bf16 and kept as fp32), a bf16 copy, and inv[r] = rsqrt(mean(x^2) + eps).
__global__ void prep_rows_kernel(const float* __restrict__ in, const uint32_t* __restrict__ rows, uint32_t k, float eps, float* out_f32,
                                 uint16_t* out_bf16, float* inv, bool normalize, bool round_out) {
    pdl_start();
    __shared__ float red[8];
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    const float* x = in + size_t(rows ? rows[r] : r) * k;
    float ss = 0.0f;
    for (uint32_t i = tid; i < k; i += 256) ss += x[i] * x[i];
    ss = warp_sum(ss);
    if (tid % 32 == 0) red[tid / 32] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (uint32_t i = 0; i < 8; i++) tot += red[i];
    const float iv = rsqrtf(tot / float(k) + eps);
    if (inv && tid == 0) inv[r] = iv;
    for (uint32_t i = tid; i < k; i += 256) {
        float v = normalize ? x[i] * iv : x[i];
        if (round_out) v = round_bf16(v);
        if (out_f32) out_f32[size_t(r) * k + i] = v;
        if (out_bf16) out_bf16[size_t(r) * k + i] = f32_to_bf16(v);
    }
}

void launch_prep_rows(const float* in, const uint32_t* rows, uint32_t n, uint32_t k, float eps, float* out_f32, uint16_t* out_bf16, float* inv,
                      bool normalize, bool round_out, cudaStream_t s) {
    if (n) launch_pdl(prep_rows_kernel, n, 256, 0, s, in, rows, k, eps, out_f32, out_bf16, inv, normalize, round_out);
}

// ------------------------------------------------------------------ sampling
// kernels.metal:1430-1451 `argmax_partial` + :1510-1576 `sample` in one kernel: each row's
// token, the argmax at temperature 0 (ties to the lowest id), else a draw from the top-p set
// by inverting the CDF of e_i = 2^((x_i - max) log2(e) / T) over a fixed order: thread t of
// 1024 owns ids t, t + 1024, ...; threads in turn. Every float operation below is a single IEEE
// operation in a fixed order, so the token is a pure function of (logit bits, seed, position).
constexpr uint32_t SAMPLE_ROUNDS = 8;

// kernels.metal:1482-1501 `tg_scan`: ex[ex_at(t)] = sum of v over threads before t,
// ex[ex_at(1024)] = the total; 32 groups of 32 threads summed left to right, then the groups.
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
        ex[ex_at(SAMPLE_THREADS)] = acc;
    }
    __syncthreads();
    ex[ex_at(tid)] = __fadd_rn(ex[ex_at(tid)], base[tid / 32]);
    __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, const SampleRow* __restrict__ rows, uint32_t* out,
                                                                const uint32_t* __restrict__ meta, uint32_t vocab, const uint32_t* __restrict__ row_skip) {
    pdl_start();
    if (row_skip && row_skip[blockIdx.x]) return;
    __shared__ float ex[SAMPLE_THREADS + SAMPLE_THREADS / 32 + 1];
    __shared__ float base[32];
    __shared__ float bvs[32];
    __shared__ uint32_t bis[32];
    __shared__ uint32_t pick;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid % 32;
    const SampleRow row = rows[r];
    const uint32_t pos = row.tok == NO_TOK ? row.pos : meta[2 * row.tok + 1] + 1;
    const float* x = logits + size_t(r) * vocab;
    float lmax = -FLT_MAX;
    uint32_t tok = 0xffffffffu;
    // A thread's ids in batches of 8: the loads of a batch go out together (a row comes from L2, and one load
    // at a time leaves the pass bound by its latency); the arithmetic keeps the id order.
    constexpr uint32_t B = 8;
    uint32_t i0 = tid;
    for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
        float v[B];
#pragma unroll
        for (uint32_t k = 0; k < B; k++) v[k] = x[i0 + k * SAMPLE_THREADS];
#pragma unroll
        for (uint32_t k = 0; k < B; k++) better(lmax, tok, v[k], i0 + k * SAMPLE_THREADS);
    }
    for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) better(lmax, tok, x[i], i);
    warp_best(lmax, tok);
    if (lane == 0) { bvs[tid / 32] = lmax; bis[tid / 32] = tok; }
    __syncthreads();
    lmax = bvs[0];
    tok = bis[0];
    for (uint32_t i = 1; i < 32; i++) better(lmax, tok, bvs[i], bis[i]);
    if (row.temperature > 0.0f) {
        const float c = __fdiv_rn(LOG2E, row.temperature);
        float s = 0.0f;
        i0 = tid;
        for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
            float v[B];
#pragma unroll
            for (uint32_t k = 0; k < B; k++) v[k] = x[i0 + k * SAMPLE_THREADS];
#pragma unroll
            for (uint32_t k = 0; k < B; k += 2) {  // the exponentials two at a time, the additions in id order
                const float2 e = soft_exp2_scaled_x2(v[k], v[k + 1], lmax, c);
                s = __fadd_rn(__fadd_rn(s, e.x), e.y);
            }
        }
        for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) s = __fadd_rn(s, soft_exp2(__fmul_rn(__fsub_rn(x[i], lmax), c)));
        tg_scan(s, ex, base, tid);
        const float z = ex[ex_at(SAMPLE_THREADS)];
        float low = -INFINITY;
        for (uint32_t round = 0; round < SAMPLE_ROUNDS; round++) {
            const float target = __fmul_rn(uniform01(row.seed_lo, row.seed_hi, pos, round), ex[ex_at(SAMPLE_THREADS)]);
            if (tid == 0) pick = 0xffffffffu;
            __syncthreads();
            const float lo = ex[ex_at(tid)];
            // The one thread whose interval holds the target re-adds its terms in order until they pass it
            // (kernels.metal:1540-1559). Its warp helps: the lanes fetch and exponentiate 32 of its ids at a time, and
            // only the additions stay in the thread's order.
            const bool mine = lo <= target && target < ex[ex_at(tid + 1)];
            const uint32_t owners = __ballot_sync(0xffffffffu, mine);
            if (owners) {
                const int src = __ffs(owners) - 1;
                const uint32_t first = __shfl_sync(0xffffffffu, tid, src);
                const float rest = __fsub_rn(target, __shfl_sync(0xffffffffu, lo, src));
                float acc = 0.0f;
                uint32_t j = 0xffffffffu;
                bool done = false;
                for (uint32_t i0w = first; i0w < vocab && !done; i0w += 32 * SAMPLE_THREADS) {
                    const uint32_t i = i0w + lane * SAMPLE_THREADS;
                    float e = 0.0f;
                    bool live = false;
                    if (i < vocab) {
                        const float xi = x[i];
                        if (xi > low) { e = soft_exp2(__fmul_rn(__fsub_rn(xi, lmax), c)); live = true; }
                    }
                    const uint32_t lives = __ballot_sync(0xffffffffu, live);
                    for (uint32_t l = 0; l < 32 && !done; l++) {
                        const float el = __shfl_sync(0xffffffffu, e, l);
                        if (!((lives >> l) & 1u)) continue;
                        acc = __fadd_rn(acc, el);
                        if (el > 0.0f) j = i0w + l * SAMPLE_THREADS;
                        if (rest < acc) done = true;
                    }
                }
                if (int(lane) == src) pick = j;
            }
            __syncthreads();
            const uint32_t j = pick;
            if (j == 0xffffffffu) break;
            const float xj = x[j];
            if (xj == lmax || row.top_p >= 1.0f) { tok = j; break; }
            float q = 0.0f;
            i0 = tid;
            for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
                float v[B];
#pragma unroll
                for (uint32_t k = 0; k < B; k++) v[k] = x[i0 + k * SAMPLE_THREADS];
#pragma unroll
                for (uint32_t k = 0; k < B; k += 2) {
                    const float2 e = soft_exp2_scaled_x2(v[k], v[k + 1], lmax, c);
                    if (v[k] > xj) q = __fadd_rn(q, e.x);
                    if (v[k + 1] > xj) q = __fadd_rn(q, e.y);
                }
            }
            for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) {
                const float xi = x[i];
                if (xi > xj) q = __fadd_rn(q, soft_exp2(__fmul_rn(__fsub_rn(xi, lmax), c)));
            }
            tg_scan(q, ex, base, tid);
            if (ex[ex_at(SAMPLE_THREADS)] < __fmul_rn(row.top_p, z)) { tok = j; break; }
            low = xj;
        }
    }
    if (tid == 0) out[r] = tok;
}

// The same sampler spread over a cluster of 8 blocks: the 1024 "threads" of the reference's order are the
// cluster's 8 x 128, so every sum keeps its order and its association (thread t still owns ids t, t + 1024,
// ...; groups of 32 threads are warps; the 32 group totals are scanned left to right), while a row's passes
// over the logits run on eight SMs instead of one. What one block needs from the others -- the best
// (value, id) pairs, the group totals, the picked id -- crosses distributed shared memory around a cluster
// barrier. Every block of a cluster takes the same branches (they hold the same values).
// STAGED: the first pass leaves this block's share of the row in shared memory ([id / 1024][thread], 512 bytes per 1024
// ids) and the later passes -- above all the one thread that walks its ids one by one to find the token -- read it there
// instead of waiting for L2 at every step.
template <bool STAGED>
__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS) sample_cluster_kernel(const float* __restrict__ logits, const SampleRow* __restrict__ rows,
                                                                                                 uint32_t* out, const uint32_t* __restrict__ meta, uint32_t vocab, const uint32_t* __restrict__ row_skip) {
    pdl_start();
    if (row_skip && row_skip[blockIdx.x / SC_CTAS]) return;  // the whole cluster leaves: no cluster barrier has been entered
    __shared__ ScExchange xc;
    __shared__ float vals[SC_THREADS], pre[SC_THREADS], tot_all[32], base[33];
    __shared__ float wbv[SC_WARPS];
    __shared__ uint32_t wbi[SC_WARPS];
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const uint32_t r = blockIdx.x / SC_CTAS, tid = threadIdx.x, lane = tid % 32, vt = rank * SC_THREADS + tid;
    const SampleRow row = rows[r];
    const uint32_t pos = row.tok == NO_TOK ? row.pos : meta[2 * row.tok + 1] + 1;
    const float* x = logits + size_t(r) * vocab;
    extern __shared__ float sc_row[];
    auto own = [&](uint32_t i) { return STAGED ? sc_row[(i / SAMPLE_THREADS) * SC_THREADS + tid] : x[i]; };  // for this thread's ids only
    constexpr uint32_t B = 8;  // a thread's ids in batches: the loads of a batch go out together, the arithmetic keeps the id order
    float lmax = -FLT_MAX;
    uint32_t tok = 0xffffffffu;
    constexpr uint32_t B1 = STAGED ? 32 : B;  // the pass that reads global memory: few threads per row, so many loads each
    uint32_t i0 = vt;
    for (; i0 + (B1 - 1) * SAMPLE_THREADS < vocab; i0 += B1 * SAMPLE_THREADS) {
        float v[B1];
#pragma unroll
        for (uint32_t k = 0; k < B1; k++) v[k] = x[i0 + k * SAMPLE_THREADS];
#pragma unroll
        for (uint32_t k = 0; k < B1; k++) {
            if (STAGED) sc_row[((i0 + k * SAMPLE_THREADS) / SAMPLE_THREADS) * SC_THREADS + tid] = v[k];
            better(lmax, tok, v[k], i0 + k * SAMPLE_THREADS);
        }
    }
    for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
        float v[B];
#pragma unroll
        for (uint32_t k = 0; k < B; k++) v[k] = x[i0 + k * SAMPLE_THREADS];
#pragma unroll
        for (uint32_t k = 0; k < B; k++) {
            if (STAGED) sc_row[((i0 + k * SAMPLE_THREADS) / SAMPLE_THREADS) * SC_THREADS + tid] = v[k];
            better(lmax, tok, v[k], i0 + k * SAMPLE_THREADS);
        }
    }
    for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) {
        const float xi = x[i];
        if (STAGED) sc_row[(i / SAMPLE_THREADS) * SC_THREADS + tid] = xi;
        better(lmax, tok, xi, i);
    }
    warp_best(lmax, tok);
    if (lane == 0) { wbv[tid / 32] = lmax; wbi[tid / 32] = tok; }
    if (tid == 0) { xc.pick[0] = NO_TOK; xc.pick[1] = NO_TOK; }
    __syncthreads();
    if (tid == 0) {
        for (uint32_t w = 1; w < SC_WARPS; w++) better(lmax, tok, wbv[w], wbi[w]);
        xc.bv = lmax;
        xc.bi = tok;
    }
    sc_cluster_sync();
    lmax = -FLT_MAX;
    tok = 0xffffffffu;
    for (uint32_t s = 0; s < SC_CTAS; s++)  // `better` is a total order on (value, id): any order of combination gives the same pair
        better(lmax, tok, __uint_as_float(sc_ld_u32(sc_remote(&xc.bv, s))), sc_ld_u32(sc_remote(&xc.bi, s)));
    if (row.temperature > 0.0f) {
        const float c = __fdiv_rn(LOG2E, row.temperature);
        float sum = 0.0f;
        i0 = vt;
        for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
            float v[B];
#pragma unroll
            for (uint32_t k = 0; k < B; k++) v[k] = own(i0 + k * SAMPLE_THREADS);
#pragma unroll
            for (uint32_t k = 0; k < B; k += 2) {
                const float2 e = soft_exp2_scaled_x2(v[k], v[k + 1], lmax, c);
                sum = __fadd_rn(__fadd_rn(sum, e.x), e.y);
            }
        }
        for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) sum = __fadd_rn(sum, soft_exp2(__fmul_rn(__fsub_rn(own(i), lmax), c)));
        float lo, hi, total;
        uint32_t scans = 0;
        sc_scan(sum, scans++ & 1, &xc, vals, pre, tot_all, base, rank, tid, lo, hi, total);
        const float z = total;
        float low = -INFINITY;
        for (uint32_t round = 0; round < SAMPLE_ROUNDS; round++) {
            const float target = __fmul_rn(uniform01(row.seed_lo, row.seed_hi, pos, round), total);
            const uint32_t pb = round & 1;
            // At most one thread of the cluster owns the target (the scan never decreases); its warp helps it as in
            // sample_kernel: 32 of its ids at a time, the additions in the thread's order.
            const uint32_t owners = __ballot_sync(0xffffffffu, lo <= target && target < hi);
            if (owners) {
                const int src = __ffs(owners) - 1;
                const uint32_t first = __shfl_sync(0xffffffffu, vt, src), col = __shfl_sync(0xffffffffu, tid, src);
                const float rest = __fsub_rn(target, __shfl_sync(0xffffffffu, lo, src));
                float acc = 0.0f;
                uint32_t j = 0xffffffffu;
                bool done = false;
                for (uint32_t i0w = first; i0w < vocab && !done; i0w += 32 * SAMPLE_THREADS) {
                    const uint32_t i = i0w + lane * SAMPLE_THREADS;
                    float e = 0.0f;
                    bool live = false;
                    if (i < vocab) {
                        const float xi = STAGED ? sc_row[(i / SAMPLE_THREADS) * SC_THREADS + col] : x[i];
                        if (xi > low) { e = soft_exp2(__fmul_rn(__fsub_rn(xi, lmax), c)); live = true; }
                    }
                    const uint32_t lives = __ballot_sync(0xffffffffu, live);
                    for (uint32_t l = 0; l < 32 && !done; l++) {
                        const float el = __shfl_sync(0xffffffffu, e, l);
                        if (!((lives >> l) & 1u)) continue;
                        acc = __fadd_rn(acc, el);
                        if (el > 0.0f) j = i0w + l * SAMPLE_THREADS;
                        if (rest < acc) done = true;
                    }
                }
                if (int(lane) == src) xc.pick[pb] = j;
            }
            sc_cluster_sync();
            uint32_t j = NO_TOK;
            for (uint32_t s = 0; s < SC_CTAS; s++) {
                const uint32_t pj = sc_ld_u32(sc_remote(&xc.pick[pb], s));
                if (pj != NO_TOK) j = pj;
            }
            if (j == NO_TOK) break;
            __syncthreads();                       // every thread of this block has read this round's picks ...
            if (tid == 0) xc.pick[pb ^ 1] = NO_TOK;  // ... of the buffer the round after next reuses; the next round's is cleared here
            const float xj = x[j];
            if (xj == lmax || row.top_p >= 1.0f) { tok = j; break; }
            float q = 0.0f;
            i0 = vt;
            for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
                float v[B];
#pragma unroll
                for (uint32_t k = 0; k < B; k++) v[k] = own(i0 + k * SAMPLE_THREADS);
#pragma unroll
                for (uint32_t k = 0; k < B; k += 2) {
                    const float2 e = soft_exp2_scaled_x2(v[k], v[k + 1], lmax, c);
                    if (v[k] > xj) q = __fadd_rn(q, e.x);
                    if (v[k + 1] > xj) q = __fadd_rn(q, e.y);
                }
            }
            for (uint32_t i = i0; i < vocab; i += SAMPLE_THREADS) {
                const float xi = own(i);
                if (xi > xj) q = __fadd_rn(q, soft_exp2(__fmul_rn(__fsub_rn(xi, lmax), c)));
            }
            sc_scan(q, scans++ & 1, &xc, vals, pre, tot_all, base, rank, tid, lo, hi, total);
            if (total < __fmul_rn(row.top_p, z)) { tok = j; break; }
            low = xj;
        }
    }
    if (rank == 0 && tid == 0) out[r] = tok;
    sc_cluster_sync();  // nobody leaves while another block may still read its shared memory
}

void launch_sample(const float* logits, const SampleRow* rows, uint32_t* out, const uint32_t* meta, uint32_t n_rows, uint32_t vocab, cudaStream_t s,
                   const uint32_t* row_skip) {
    if (!n_rows) return;
    // Enough rows to fill the SMs with one block each: the single-block form (at 160 rows the two take the same time,
    // bound by instruction issue); fewer: a cluster of 8 blocks per row (one stream's 5 rows: 95 -> about 25 us).
    if (n_rows > 96) { launch_pdl(sample_kernel, n_rows, SAMPLE_THREADS, 0, s, logits, rows, out, meta, vocab, row_skip); return; }
    // A block's share of a row in shared memory (512 bytes per 1024 ids), if it fits.
    const size_t stage = size_t((vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS) * SC_THREADS * 4;
    const bool staged = stage <= 200 * 1024;
    static PerDevice configured;
    configured.once([] { VLT_CUDA(cudaFuncSetAttribute(sample_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); });
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_rows * SC_CTAS);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = staged ? stage : 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (staged) VLT_CUDA(cudaLaunchKernelEx(&cfg, sample_cluster_kernel<true>, logits, rows, out, meta, vocab, row_skip));
    else VLT_CUDA(cudaLaunchKernelEx(&cfg, sample_cluster_kernel<false>, logits, rows, out, meta, vocab, row_skip));
    launch_counter()++;
}

// ----------------------------------------------------------------- accepting
// kernels.metal:1605-1657 `accept`: what each run emits and how far its sequence advances.
// One thread per run.
__global__ void accept_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ tokens, uint32_t* out, uint32_t* lens, uint32_t* feed,
                              GenState* gen, uint32_t* emitted, uint32_t nruns, const uint32_t* __restrict__ tree, uint32_t* path,
                              uint32_t* path_len, uint32_t* on_path, const uint32_t* __restrict__ spec_e) {
    pdl_start();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nruns) return;
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
    const uint32_t decided = ru.verify && spec_e ? min(spec_e[r], ru.count) : 0u;
    if (decided) {
        // The rejection-sampling rule settled this run's candidates (k_spec.cu): rows 0 .. decided - 1 are the path.
        e = decided;
        for (uint32_t j = 0; j < e; j++) walk[j] = j;
        first = ru.head0;
    } else if (ru.verify) {
        // Children come after their parents, so one pass over the rows finds the path.
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

void launch_accept(const RunIn* runs, const uint32_t* tokens, uint32_t* out, uint32_t* lens, uint32_t* feed, GenState* gen, uint32_t* emitted,
                   uint32_t n_runs, const uint32_t* tree, uint32_t* path, uint32_t* path_len, uint32_t* on_path, cudaStream_t s, const uint32_t* spec_e) {
    if (n_runs) launch_pdl(accept_kernel, (n_runs + 63) / 64, 64, 0, s, runs, tokens, out, lens, feed, gen, emitted, n_runs, tree, path, path_len, on_path, spec_e);
}

// kernels.metal:1663-1693 `kv_compact`: the accepted path's K/V rows, on every layer, from
// p0 + path[j] to p0 + j. grid (runs, layers); a warp per kv head, a lane per pair of dims.
__global__ void kv_compact_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ path, const uint32_t* __restrict__ path_len,
                                  const uint32_t* __restrict__ lens, uint16_t* k_cache, uint16_t* v_cache, const uint32_t* __restrict__ page_table,
                                  KvArgs kv) {
    pdl_start();
    const uint32_t r = blockIdx.x, l = blockIdx.y, g = threadIdx.x / 32, lane = threadIdx.x % 32, k = path_len[r];
    const uint32_t slot = runs[r].slot, p0 = lens[slot] - k;
    for (uint32_t j = 1; j < k; j++) {
        const uint32_t from = path[r * FEED_W + j];
        if (from == j) continue;
        const size_t src = kv_row(kv, l, page_table, slot, g, p0 + from), dst = kv_row(kv, l, page_table, slot, g, p0 + j);
        reinterpret_cast<uint32_t*>(k_cache + dst)[lane] = reinterpret_cast<const uint32_t*>(k_cache + src)[lane];
        reinterpret_cast<uint32_t*>(v_cache + dst)[lane] = reinterpret_cast<const uint32_t*>(v_cache + src)[lane];
    }
}

void launch_kv_compact(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* lens, uint16_t* k_cache, uint16_t* v_cache,
                       const uint32_t* page_table, KvArgs kv, uint32_t n_runs, uint32_t n_layers, cudaStream_t s) {
    if (n_runs) launch_pdl(kv_compact_kernel, dim3(n_runs, n_layers), 32 * kv.n_kv, 0, s, runs, path, path_len, lens, k_cache, v_cache, page_table, kv);
}

// kernels.metal:1705-1724 `replay_draft`. grid: runs blocks of FEED_W threads.
__global__ void replay_draft_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ lens, uint32_t* feed, const uint32_t* __restrict__ trace,
                                    const uint32_t* __restrict__ trace_len, ReplayArgs ra, uint32_t nruns, uint32_t* tree) {
    pdl_start();
    const uint32_t r = blockIdx.x, i = threadIdx.x;
    if (i == 0 || i >= FEED_W || r >= nruns || runs[r].nhead == 0) return;
    const uint32_t slot = runs[r].slot, n = trace_len[slot];
    if (n == 0) return;
    const uint32_t pos = lens[slot] + i;
    uint32_t tok = pos < n ? trace[size_t(slot) * ra.stride + pos] : 0u;
    const uint32_t h = philox(make_uint4(pos, 0x5eed, 0, 0), ra.seed, 0x0dd5u).x;
    if (__fmul_rn(float(h >> 8), 0x1p-24f) < ra.rate) tok = (tok + 1) % ra.vocab;
    feed[slot * FEED_W + i] = tok;
    tree[slot * FEED_W + i] = d_chain_node(i);
}

void launch_replay_draft(const RunIn* runs, const uint32_t* lens, uint32_t* feed, const uint32_t* trace, const uint32_t* trace_len, ReplayArgs ra,
                         uint32_t n_runs, uint32_t* tree, cudaStream_t s) {
    if (n_runs) launch_pdl(replay_draft_kernel, n_runs, FEED_W, 0, s, runs, lens, feed, trace, trace_len, ra, n_runs, tree);
}

// A wait that runs out, by design of the wait: one warp polls an mbarrier that expects an arrival nobody makes, gives up
// after `polls` tries -- the same bounded wait every kernel here uses around its copies -- and reports it the same way, in
// the device error word. Nothing faults or hangs; the kernel returns. Exists so that the reporting path (the error word
// travelling down with a step's results, the step raising, the engine carrying on) can be tested.
__global__ void stalled_wait_kernel(uint32_t* err_flag, uint32_t polls, uint32_t code) {
    __shared__ uint64_t bar;
    const uint32_t addr = uint32_t(__cvta_generic_to_shared(&bar));
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(1u));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    bool arrived = false;
    for (uint32_t i = 0; i < polls && !arrived; i++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(addr), "r"(0u) : "memory");
        arrived = ok != 0;
    }
    if (!arrived && threadIdx.x == 0) atomicExch(err_flag, code);
}
void launch_stalled_wait(uint32_t* err_flag, uint32_t polls, uint32_t code, cudaStream_t s) {
    stalled_wait_kernel<<<1, 32, 0, s>>>(err_flag, polls, code);
    launch_counter()++;
}

// bench_fill's optional K/V values: small pseudo-random bf16 numbers (a hash of seed, layer,
// head, position and dim) at positions [from, to) of a slot, so that timing runs read finite data.
__global__ void kv_fill_kernel(uint16_t* k_cache, uint16_t* v_cache, const uint32_t* __restrict__ page_table, KvArgs kv, uint32_t slot, uint32_t from,
                               uint32_t to, uint32_t seed) {
    const uint32_t layer = blockIdx.y, g = blockIdx.z;
    for (uint32_t pos = from + blockIdx.x; pos < to; pos += gridDim.x) {
        const size_t at = kv_row(kv, layer, page_table, slot, g, pos);
        const uint32_t d = threadIdx.x;  // a pair of dims
        const uint4 h = philox(make_uint4(pos, layer * 64 + g, d, slot), seed, 0x6b76u);
        auto val = [](uint32_t u) { return (float(u >> 8) * 0x1p-24f - 0.5f) * 2.0f; };
        reinterpret_cast<uint32_t*>(k_cache + at)[d] = pack_bf16(val(h.x), val(h.y));
        reinterpret_cast<uint32_t*>(v_cache + at)[d] = pack_bf16(val(h.z), val(h.w));
    }
}

void launch_kv_fill(uint16_t* k_cache, uint16_t* v_cache, const uint32_t* page_table, KvArgs kv, uint32_t n_layers, uint32_t slot, uint32_t from,
                    uint32_t to, uint32_t seed, cudaStream_t s) {
    if (to <= from) return;
    const uint32_t blocks = std::min(to - from, 1024u);
    { kv_fill_kernel<<<dim3(blocks, n_layers, kv.n_kv), kv.hd / 2, 0, s>>>(k_cache, v_cache, page_table, kv, slot, from, to, seed); launch_counter()++; }
}

}  // namespace vlt
