// The reference's own architecture (engine/src/model.rs, engine/src/engine/encode.rs:99-192): what its layers do beyond
// a plain decoder's, as small kernels of their own. The projections are the engine's streamed matmul and tensor-core GEMM
// with the matrix scales and residual lambdas in their epilogues. Here: `mudd` (kernels.metal:1364-1407), the per-token work after the qkv
// projection (`qkv_post` / `new_key`, :725-801,910-945: q/k RMS-norm per head of 128, RoPE on the first 64 dims of local
// layers, gated value embeddings, K/V rounded into a ring per (local layer, slot) or into the paged pool of the global
// layers, XSA directions, attention gates), the merge of the attention's key splits with XSA and the gate applied
// (`attn_dec_reduce`, :1314-1362; the attention itself is k_limite_attn.cu, and a one-block form of it here serves kv
// heads with more than eight query heads), and the path compaction over both kinds of cache (`kv_compact`, :1663-1693).
#include <algorithm>
#include <cfloat>

#include "kernels.h"

namespace vlt {

namespace limite {

constexpr uint32_t D = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
// kernels.metal:31-38: erf by Abramowitz & Stegun 7.1.26, and gelu over it.
__device__ __forceinline__ float erf_as(float x) {
    const float a = fabsf(x), t = 1.0f / (1.0f + 0.3275911f * a);
    const float y = 1.0f - (((((1.061405429f * t - 1.453152027f) * t) + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t * expf(-a * a);
    return copysignf(y, x);
}
__device__ __forceinline__ float gelu(float x) { return 0.5f * x * (1.0f + erf_as(x * 0.70710678118654752f)); }

// kernels.metal:704-715 `kv_row_of`: where kv head g's row of cache position pos starts (in elements).
__device__ __forceinline__ size_t kv_row(const LimiteKv& kv, uint32_t slot, uint32_t g, uint32_t pos) {
    if (kv.is_global) {
        const uint32_t page = kv.page_table[size_t(slot) * kv.max_pages + (pos >> kv.page_shift)], psize = 1u << kv.page_shift;
        return ((size_t(kv.layer) * kv.n_pages + page) * kv.n_kv + g) * psize * D + size_t(pos & (psize - 1)) * D;
    }
    return ((size_t(kv.layer) * kv.max_seqs + slot) * kv.n_kv + g) * kv.ring * D + size_t(pos % kv.ring) * D;
}

// kernels.metal:727-736 `norm_rope` for a warp that holds a head (lane: dims 4 lane .. 4 lane + 3).
__device__ __forceinline__ float4 norm_rope(float4 v, bool rope, float eps, uint32_t lane, const float2* cs) {
    const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    const float inv = 1.0f / sqrtf(ss / float(D) + eps);
    v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
    if (rope && lane < 16) {
        const float2 c0 = cs[2 * lane], c1 = cs[2 * lane + 1];
        const float a0 = v.x, a1 = v.y, b0 = v.z, b1 = v.w;
        v = make_float4(c0.x * a0 + c0.y * a1, c0.x * a1 - c0.y * a0, c1.x * b0 + c1.y * b1, c1.x * b1 - c1.y * b0);
    }
    return v;
}

// kernels.metal:1364-1407 `mudd`: one inner projection of rms_norm(current) feeds two mixes of (tap0, tap1, current) --
// the attention's input and the residual base. One block of 256 threads per token.
__global__ void mudd_kernel(const float* __restrict__ cur, const float* __restrict__ tap0, const float* __restrict__ tap1, const float* __restrict__ dense1,
                            const float* __restrict__ mix, uint32_t hidden, float eps, float* out_attn, float* out_base) {
    pdl_start();
    __shared__ float red[8], inner[32], w[6];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const float* c = cur + size_t(t) * hidden;
    float ss = 0.0f;
    for (uint32_t i = tid; i < hidden; i += 256) ss += c[i] * c[i];
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < 8; i++) total += red[i];
    const float inv = 1.0f / sqrtf(total / float(hidden) + eps);
    for (uint32_t j = warp * 4; j < warp * 4 + 4; j++) {
        float s = 0.0f;
        for (uint32_t k = lane; k < hidden; k += 32) s += c[k] * inv * dense1[size_t(j) * hidden + k];
        s = warp_sum(s);
        if (lane == 0) inner[j] = gelu(s);
    }
    __syncthreads();
    if (tid < 6) {
        const float* row = mix + tid * 33;
        float s = 0.0f;
        for (uint32_t j = 0; j < 32; j++) s += inner[j] * row[j];
        w[tid] = s + row[32];
    }
    __syncthreads();
    for (uint32_t i = tid; i < hidden; i += 256) {
        const size_t o = size_t(t) * hidden + i;
        const float a = tap0[o], b = tap1[o], x = c[i];
        out_attn[o] = w[0] * a + w[1] * b + w[2] * x;
        out_base[o] = w[3] * a + w[4] * b + w[5] * x;
    }
}

// After the qkv projection, one block per token, a warp per head (query heads, then kv heads). x: the attention's input
// before its norm; its 1 / rms from inv_rms, or (inv_rms null) from ssq.
__global__ void qkv_post_kernel(float* qkv, const float* __restrict__ x, const float* __restrict__ inv_rms, const uint32_t* __restrict__ meta,
                                const uint32_t* __restrict__ tin, const uint32_t* __restrict__ tokens, const uint16_t* __restrict__ ve_table,
                                const float* __restrict__ ve_gate, const float* __restrict__ attn_gate, const float* __restrict__ rope, const LimiteKv kv,
                                uint32_t hidden, uint32_t n_q, float eps, uint32_t vocab, uint16_t* k_cache, uint16_t* v_cache, float* vdir, float* gates,
                                const float* __restrict__ ssq, uint32_t ssq_tiles, uint32_t ssq_stride) {
    pdl_start();
    const uint32_t t = blockIdx.x, w = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], row = tin[2 * t + 1], qw = (n_q + 2 * kv.n_kv) * D;
    float inv;
    if (inv_rms) inv = inv_rms[t];
    else {  // the sums of squares the GEMM before left per 128-row tile, as the qkv GEMM itself takes them
        float ss = 0.0f;
        for (uint32_t tl = 0; tl < ssq_tiles; tl++) ss += ssq[size_t(tl) * ssq_stride + t];
        inv = rsqrtf(ss / float(hidden) + eps);
    }
    const float* xt = x + size_t(t) * hidden;
    const float2* cs = reinterpret_cast<const float2*>(rope) + size_t(pos) * 32;
    const bool turn = !kv.is_global;  // encode.rs:227: global layers take no RoPE
    if (w < n_q) {
        float* q = qkv + size_t(t) * qw + w * D + d0;
        *reinterpret_cast<float4*>(q) = norm_rope(*reinterpret_cast<const float4*>(q), turn, eps, lane, cs);
        // The attention gate: 2 sigmoid(rms_norm(x)[:128] . attn_gate[h]), kernels.metal:781-784.
        const float4 xg = *reinterpret_cast<const float4*>(xt + d0), ag = *reinterpret_cast<const float4*>(attn_gate + w * D + d0);
        const float s = warp_sum((xg.x * ag.x + xg.y * ag.y + xg.z * ag.z + xg.w * ag.w) * inv);
        if (lane == 0) gates[size_t(t) * n_q + w] = 2.0f * sigmoid(s);
        return;
    }
    const uint32_t g = w - n_q;
    float* kp = qkv + size_t(t) * qw + (n_q + g) * D + d0;
    float* vp = qkv + size_t(t) * qw + (n_q + kv.n_kv + g) * D + d0;
    const float4 kk = norm_rope(*reinterpret_cast<const float4*>(kp), turn, eps, lane, cs);
    float4 vv = *reinterpret_cast<const float4*>(vp);
    if (ve_gate) {  // kernels.metal:738-747 `add_ve`: v + 2 sigmoid(rms_norm(x)[:12] . ve_gate[g]) value_embed[token][g]
        float s = 0.0f;
        if (lane < 3) {
            const float4 xg = *reinterpret_cast<const float4*>(xt + d0), vg = *reinterpret_cast<const float4*>(ve_gate + g * 12 + d0);
            s = (xg.x * vg.x + xg.y * vg.y + xg.z * vg.z + xg.w * vg.w) * inv;
        }
        const float gate = 2.0f * sigmoid(warp_sum(s));
        uint32_t tok = tokens[t];
        if (tok >= vocab) tok = 0;
        const uint2 ve = *reinterpret_cast<const uint2*>(ve_table + size_t(tok) * kv.n_kv * D + g * D + d0);
        vv.x += gate * bf16lo(ve.x); vv.y += gate * bf16hi(ve.x); vv.z += gate * bf16lo(ve.y); vv.w += gate * bf16hi(ve.y);
    }
    *reinterpret_cast<float4*>(kp) = kk;
    *reinterpret_cast<float4*>(vp) = vv;
    const uint32_t cpos = meta[2 * (t - row) + 1] + row;  // kernels.metal:74-77 `cache_pos`
    const size_t at = kv_row(kv, slot, g, cpos) + d0;
    *reinterpret_cast<uint2*>(k_cache + at) = make_uint2(pack_bf16(kk.x, kk.y), pack_bf16(kk.z, kk.w));
    *reinterpret_cast<uint2*>(v_cache + at) = make_uint2(pack_bf16(vv.x, vv.y), pack_bf16(vv.z, vv.w));
    const float nrm = fmaxf(sqrtf(warp_sum(vv.x * vv.x + vv.y * vv.y + vv.z * vv.z + vv.w * vv.w)), 1e-4f);  // XSA_EPS
    *reinterpret_cast<float4*>(vdir + (size_t(t) * kv.n_kv + g) * D + d0) = make_float4(vv.x / nrm, vv.y / nrm, vv.z / nrm, vv.w / nrm);
}

// A row's attention, grid (tokens, query heads), four warps: the cached keys from the row's window start (0 on a global
// layer) up to its tile's first position, then the tile's rows its `vis` names (at most 8, at the tile's first position
// + their row: siblings of a draft tree share positions but not cache rows). A warp takes every fourth key, a lane four
// of the 128 dims; online softmax per warp, merged through shared memory; then XSA -- the output minus xsa[h] times its
// projection on the token's value direction -- and the head's gate (`attn_dec_reduce`).
__global__ void attn_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ vis,
                            const uint16_t* __restrict__ k_cache, const uint16_t* __restrict__ v_cache, const LimiteKv kv, uint32_t n_q, uint32_t window, float scale,
                            const float* __restrict__ vdir, const float* __restrict__ gates, const float* __restrict__ xsa, float* out) {
    pdl_start();
    __shared__ float ms[4], ls[4];
    __shared__ float os[4][D];
    const uint32_t t = blockIdx.x, h = blockIdx.y, w = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], row = tin[2 * t + 1], mask = vis[t];
    const uint32_t p0 = meta[2 * (t - row % 8) + 1], lo = kv.is_global ? 0u : (pos > window ? pos - window : 0u);  // kernels.metal:809 `key_lo`
    const uint32_t p_run = meta[2 * (t - row) + 1] + (row - row % 8);  // the cache position of the tile's first row
    const uint32_t g = h / (n_q / kv.n_kv), qw = (n_q + 2 * kv.n_kv) * D;
    const float4 q = *reinterpret_cast<const float4*>(qkv + size_t(t) * qw + h * D + d0);
    float m = -INFINITY, l = 0.0f;
    float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const uint32_t n_old = p0 > lo ? p0 - lo : 0;
    for (uint32_t i = w; i < n_old + 8; i += 4) {
        uint32_t kp;
        if (i < n_old) kp = lo + i;
        else if ((mask >> (i - n_old)) & 1u) kp = p_run + (i - n_old);
        else continue;
        const size_t at = kv_row(kv, slot, g, kp) + d0;
        const uint2 kb = *reinterpret_cast<const uint2*>(k_cache + at), vb = *reinterpret_cast<const uint2*>(v_cache + at);
        const float s = warp_sum(q.x * bf16lo(kb.x) + q.y * bf16hi(kb.x) + q.z * bf16lo(kb.y) + q.w * bf16hi(kb.y)) * scale;
        const float mn = fmaxf(m, s), corr = __expf(m - mn), p = __expf(s - mn);
        l = l * corr + p;
        o.x = o.x * corr + p * bf16lo(vb.x);
        o.y = o.y * corr + p * bf16hi(vb.x);
        o.z = o.z * corr + p * bf16lo(vb.y);
        o.w = o.w * corr + p * bf16hi(vb.y);
        m = mn;
    }
    if (lane == 0) { ms[w] = m; ls[w] = l; }
    *reinterpret_cast<float4*>(&os[w][d0]) = o;
    __syncthreads();
    const float mm = fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3]));
    float ll = 0.0f;
    float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float wk = ms[k] == -INFINITY ? 0.0f : __expf(ms[k] - mm);
        const float4 ok = *reinterpret_cast<const float4*>(&os[k][d0]);
        ll += ls[k] * wk;
        oo.x += ok.x * wk; oo.y += ok.y * wk; oo.z += ok.z * wk; oo.w += ok.w * wk;
    }
    oo.x /= ll; oo.y /= ll; oo.z /= ll; oo.w /= ll;
    // Every warp holds the same oo now (each computed it from shared memory); warp 0 finishes.
    if (w) return;
    const float4 vd = *reinterpret_cast<const float4*>(vdir + (size_t(t) * kv.n_kv + g) * D + d0);
    const float pr = warp_sum(oo.x * vd.x + oo.y * vd.y + oo.z * vd.z + oo.w * vd.w);
    const float xs = xsa[h] * pr, gt = gates[size_t(t) * n_q + h];
    *reinterpret_cast<float4*>(out + (size_t(t) * n_q + h) * D + d0) = make_float4((oo.x - xs * vd.x) * gt, (oo.y - xs * vd.y) * gt, (oo.z - xs * vd.z) * gt, (oo.w - xs * vd.w) * gt);
}

constexpr uint32_t PART = 132;  // floats per partial: m, l, 2 pad, o[128] (kernels.metal:15)

// The splits' partials of a (token, head) added up (an empty split has m = -inf), then XSA and the gate
// (kernels.metal:1314-1362 `attn_dec_reduce`). grid (tokens, heads), four warps: warp w takes splits w, w + 4, ..., eight
// at a time with their loads together (one after the other each is an L2 round trip, and there are up to 128); the warps'
// sums meet in shared memory.
__global__ void __launch_bounds__(128) merge_kernel(const float* __restrict__ part, uint32_t max_splits, uint32_t n_q, uint32_t n_kv, const float* __restrict__ vdir,
                                                    const float* __restrict__ gates, const float* __restrict__ xsa, float* out, uint16_t* out_b) {
    pdl_start();
    __shared__ float ms[4], ls[4];
    __shared__ float os[4][D];
    const uint32_t t = blockIdx.x, h = blockIdx.y, w = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane, g = h / (n_q / n_kv);
    const float* pp = part + (size_t(t) * n_q + h) * max_splits * PART;
    float m = -INFINITY, l = 0.0f;
    float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t s0 = w; s0 < max_splits; s0 += 32) {
        float2 ml[8];
        float4 ov[8];
#pragma unroll
        for (uint32_t u = 0; u < 8; u++) {
            const uint32_t sp = s0 + 4 * u;
            ml[u] = make_float2(-INFINITY, 0.0f);
            ov[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (sp < max_splits) {
                ml[u] = *reinterpret_cast<const float2*>(pp + sp * PART);
                ov[u] = *reinterpret_cast<const float4*>(pp + sp * PART + 4 + d0);
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < 8; u++) {
            if (ml[u].x == -INFINITY) continue;  // (the same for the whole warp)
            const float mn = fmaxf(m, ml[u].x), corr = __expf(m - mn), wk = __expf(ml[u].x - mn);
            l = l * corr + ml[u].y * wk;
            o.x = o.x * corr + ov[u].x * wk;
            o.y = o.y * corr + ov[u].y * wk;
            o.z = o.z * corr + ov[u].z * wk;
            o.w = o.w * corr + ov[u].w * wk;
            m = mn;
        }
    }
    if (lane == 0) { ms[w] = m; ls[w] = l; }
    *reinterpret_cast<float4*>(&os[w][d0]) = o;
    __syncthreads();
    if (w) return;
    const float mm = fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3]));
    float ll = 0.0f;
    float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float wk = ms[k] == -INFINITY ? 0.0f : __expf(ms[k] - mm);
        const float4 ok = *reinterpret_cast<const float4*>(&os[k][d0]);
        ll += ls[k] * wk;
        oo.x += ok.x * wk; oo.y += ok.y * wk; oo.z += ok.z * wk; oo.w += ok.w * wk;
    }
    oo.x /= ll; oo.y /= ll; oo.z /= ll; oo.w /= ll;
    float4 r = oo;
    if (vdir) {  // (none for the block drafter's layers: no XSA, no gate)
        const float4 vd = *reinterpret_cast<const float4*>(vdir + (size_t(t) * n_kv + g) * D + d0);
        const float pr = warp_sum(oo.x * vd.x + oo.y * vd.y + oo.z * vd.z + oo.w * vd.w);
        const float xs = xsa[h] * pr, gt = gates[size_t(t) * n_q + h];
        r = make_float4((oo.x - xs * vd.x) * gt, (oo.y - xs * vd.y) * gt, (oo.z - xs * vd.z) * gt, (oo.w - xs * vd.w) * gt);
    }
    *reinterpret_cast<float4*>(out + (size_t(t) * n_q + h) * D + d0) = r;
    if (out_b) *reinterpret_cast<uint2*>(out_b + (size_t(t) * n_q + h) * D + d0) = make_uint2(pack_bf16(r.x, r.y), pack_bf16(r.z, r.w));  // for a tensor-core o projection
}

// kernels.metal:1663-1693 `kv_compact` over the local rings and the global pool. grid (runs, local + global layers), a warp
// per kv head.
__global__ void compact_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ path, const uint32_t* __restrict__ path_len, const uint32_t* __restrict__ lens,
                               uint16_t* k_local, uint16_t* v_local, uint16_t* k_global, uint16_t* v_global, LimiteKv local, LimiteKv global, uint32_t n_local) {
    pdl_start();
    const uint32_t r = blockIdx.x, l = blockIdx.y, k = path_len[r], g = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (k < 2) return;
    const uint32_t slot = runs[r].slot, p0 = lens[slot] - k;
    const bool gl = l >= n_local;
    LimiteKv kv = gl ? global : local;
    kv.layer = gl ? l - n_local : l;
    uint16_t* kc = gl ? k_global : k_local;
    uint16_t* vc = gl ? v_global : v_local;
    for (uint32_t j = 1; j < k; j++) {
        const uint32_t from = path[r * FEED_W + j];
        if (from == j) continue;
        const size_t src = kv_row(kv, slot, g, p0 + from) + lane * 4, dst = kv_row(kv, slot, g, p0 + j) + lane * 4;
        *reinterpret_cast<uint2*>(kc + dst) = *reinterpret_cast<const uint2*>(kc + src);
        *reinterpret_cast<uint2*>(vc + dst) = *reinterpret_cast<const uint2*>(vc + src);
    }
}

}  // namespace limite

void launch_limite_mudd(const float* cur, const float* tap0, const float* tap1, const float* dense1, const float* mix, uint32_t hidden, float eps, uint32_t n,
                        float* out_attn, float* out_base, cudaStream_t s) {
    launch_pdl(limite::mudd_kernel, n, 256, 0, s, cur, tap0, tap1, dense1, mix, hidden, eps, out_attn, out_base);
}
void launch_limite_qkv_post(float* qkv, const float* x, const float* inv_rms, const uint32_t* meta, const uint32_t* tin, const uint32_t* tokens, const uint16_t* ve_table,
                            const float* ve_gate, const float* attn_gate, const float* rope, const LimiteKv& kv, uint32_t hidden, uint32_t n_q, float eps, uint32_t vocab,
                            uint32_t n, uint16_t* k_cache, uint16_t* v_cache, float* vdir, float* gates, const float* ssq, uint32_t ssq_tiles, uint32_t ssq_stride,
                            cudaStream_t s) {
    launch_pdl(limite::qkv_post_kernel, n, 32 * (n_q + kv.n_kv), 0, s, qkv, x, inv_rms, meta, tin, tokens, ve_table, ve_gate, attn_gate, rope, kv, hidden, n_q, eps, vocab,
               k_cache, v_cache, vdir, gates, ssq, ssq_tiles, ssq_stride);
}
// max_keys: the most keys a row of the step may see on this layer (its tile's eight slots included); part: room for
// n * n_q * LIMITE_MAX_SPLITS partials of 132 floats (or as many splits as max_keys / 64 can make); tiles: the step's
// (first row, rows <= 8) pairs. More than 8 query heads per kv head take the one-block-per-(token, head) kernel.
void launch_limite_attn(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint32_t* tiles, uint32_t n_tiles,
                        const uint16_t* k_cache, const uint16_t* v_cache, const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, const float* vdir, const float* gates, const float* xsa, uint32_t n,
                        uint32_t max_keys, float* part, float* out, uint16_t* out_b, uint32_t keys_per_block, cudaStream_t s) {
    const uint32_t G = n_q / kv.n_kv;
    if (G > 8) {
        if (out_b || !vdir) throw Error("internal: the one-block attention leaves no bf16 copy and wants XSA directions and gates");
        launch_pdl(limite::attn_kernel, dim3(n, n_q), 128, 0, s, qkv, meta, tin, vis, k_cache, v_cache, kv, n_q, window, scale, vdir, gates, xsa, out);
        return;
    }
    // A step whose tiles hold two rows or more on average (draft trees under verification, the block drafter's blocks)
    // takes the kernel that reads a tile's keys once for all its rows; plain decoding the one that splits a row's keys
    // over four warps.
    const bool by_tile = tiles && n_tiles && n >= 2 * n_tiles && G <= 6;  // (8 rows x G heads in its 48 columns)
    // Key splits, in whole rounds of 64 keys, at most LIMITE_MAX_SPLITS. The one-row kernel (three blocks an SM, which
    // need not run in step): enough blocks to fill a B200's 148 SMs twice over. The rows' kernel (two blocks an SM): the count
    // that makes waves of blocks times a block's keys, plus a fixed part of about 128 keys' worth, least.
    const uint32_t most = std::max(1u, std::min(LIMITE_MAX_SPLITS, (max_keys + 63) / 64));
    uint32_t splits = 1;
    if (by_tile) {
        const uint32_t units = std::max(n_tiles * kv.n_kv, 1u), slots = 2 * 148;
        uint64_t best = ~0ull;
        for (uint32_t c = 1; c <= most; c++) {
            const uint32_t k = ((max_keys + c - 1) / c + 63) / 64 * 64, real = (max_keys + k - 1) / k;
            const uint64_t cost = uint64_t((units * real + slots - 1) / slots) * (k + 128);
            if (cost < best) { best = cost; splits = real; }
        }
    } else {
        const uint32_t units = std::max(n * kv.n_kv, 1u);
        splits = std::max(1u, std::min(most, (6 * 148 + units - 1) / units));
    }
    if (keys_per_block) splits = std::max(1u, std::min(LIMITE_MAX_SPLITS, (max_keys + keys_per_block - 1) / keys_per_block));  // (a tuning override)
    const uint32_t kps = ((max_keys + splits - 1) / splits + 63) / 64 * 64;
    splits = (max_keys + kps - 1) / kps;
    // Few keys (a local layer's window, a short context), rows enough to fill the SMs with at most 8 splits each, and no
    // tuning override: the splits as one thread-block cluster, which merges them itself and applies XSA and the gate -- no
    // merge kernel. (With few rows the finer splits and the second kernel are faster: 2.06 against 2.13 ms a step at one
    // stream of the reference's shapes, 2.40 against 2.45 at 8; 2.91 against 2.87 at 32.)
    if (!by_tile && vdir && !keys_per_block && max_keys <= 2048 && n * kv.n_kv >= 48) {
        const uint32_t c = std::min(splits, 8u), k = ((max_keys + c - 1) / c + 63) / 64 * 64;
        launch_limite_attn_cluster(qkv, meta, tin, vis, k_cache, v_cache, kv, n_q, window, scale, vdir, gates, xsa, n, k, (max_keys + k - 1) / k, out, out_b, s);
        return;
    }
    if (by_tile) launch_limite_attn_rows(qkv, meta, tin, vis, tiles, k_cache, v_cache, kv, n_q, window, scale, n_tiles, kps, splits, part, s);
    else launch_limite_attn_mma(qkv, meta, tin, vis, k_cache, v_cache, kv, n_q, window, scale, n, kps, splits, part, s);
    launch_pdl(limite::merge_kernel, dim3(n, n_q), 128, 0, s, part, splits, n_q, kv.n_kv, vdir, gates, xsa, out, out_b);
}
void launch_limite_compact(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* lens, uint16_t* k_local, uint16_t* v_local,
                           uint16_t* k_global, uint16_t* v_global, const LimiteKv& local, const LimiteKv& global, uint32_t n_local, uint32_t n_global, uint32_t n_runs,
                           cudaStream_t s) {
    launch_pdl(limite::compact_kernel, dim3(n_runs, n_local + n_global), 32 * local.n_kv, 0, s, runs, path, path_len, lens, k_local, v_local, k_global, v_global, local,
               global, n_local);
}

}  // namespace vlt
