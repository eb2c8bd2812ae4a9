// The reference's block drafter (engine/src/engine/drafter.rs:278-447, tools/spec/drafter.py): its own kernels. Its
// matmuls are the engine's (fc, kv_all, inject, the convolutions' corrections, qkv, o, gate_up, down, head), its
// candidates and trees k_draft.cu's draft_top / draft_tree. What is here replaces kernels.metal:1735-1840 (`draft_kv`,
// `draft_ctx`, `draft_embed`, `draft_conv`) and, for the block rows, the local-layer path of `qkv_post` and
// `attn_verify` (kernels.metal:704-736, 749-801, 808-811): q and k rms-normed per head of 128 and turned on their first
// 64 dims, keys and values in a ring per (layer, slot), a row seeing the `window` positions before it below its block,
// and its whole block. (That attention runs through k_limite_attn.cu's rows kernel when a kv head has at most six query
// heads; the kernel here serves the others.)
#include <cfloat>

#include "kernels.h"

namespace vlt {

namespace block {

constexpr uint32_t D = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// kernels.metal:727-736 `norm_rope` for a warp that holds a head (lane: dims 4 lane .. 4 lane + 3): rms_norm over the
// head, then RoPE on dims 0..63 as 32 interleaved pairs; cs: this position's (cos, sin) per pair.
__device__ __forceinline__ float4 norm_rope(float4 v, float eps, uint32_t lane, const float2* cs) {
    const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    const float inv = 1.0f / sqrtf(ss / float(D) + eps);
    v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
    if (lane < 16) {
        const float2 c0 = cs[2 * lane], c1 = cs[2 * lane + 1];
        const float a0 = v.x, a1 = v.y, b0 = v.z, b1 = v.w;
        v = make_float4(c0.x * a0 + c0.y * a1, c0.x * a1 - c0.y * a0, c1.x * b0 + c1.y * b1, c1.x * b1 - c1.y * b0);
    }
    return v;
}

__device__ __forceinline__ size_t ring_row(const BlockDrafterDims& b, uint32_t layer, uint32_t slot, uint32_t g, uint32_t pos) {  // kernels.metal:710, local
    return ((size_t(layer) * b.max_seqs + slot) * b.n_kv + g) * b.ring * D + size_t(pos % b.ring) * D;
}
__device__ __forceinline__ void store_bf16x4(uint16_t* dst, float4 v) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

// kernels.metal:1735-1774 `draft_kv` + `draft_ctx`. grid (tokens, layers + 1), 32 threads per kv head: blockIdx.y below
// the layer count writes that layer's keys (normed, turned) and values of the token into the rings; the last one the
// token's normed context into the slot's context ring. Only tokens on the accepted path.
__global__ void context_kernel(const float* __restrict__ kvp, const float* __restrict__ ctx, const float* __restrict__ ctx_inv, const uint32_t* __restrict__ meta,
                               const uint32_t* __restrict__ on_path, const float* __restrict__ rope, const BlockDrafterDims b, uint16_t* k_ring, uint16_t* v_ring,
                               float* ctx_ring) {
    pdl_start();
    const uint32_t t = blockIdx.x, l = blockIdx.y;
    if (!on_path[t]) return;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1];
    if (l == b.n_layers) {
        float* dst = ctx_ring + (size_t(slot) * b.ctx_ring_len + pos % b.ctx_ring_len) * b.hidden;
        const float inv = ctx_inv[t];
        for (uint32_t d = threadIdx.x; d < b.hidden; d += blockDim.x) dst[d] = ctx[size_t(t) * b.hidden + d] * inv;
        return;
    }
    const uint32_t g = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane;
    const float* row = kvp + (size_t(t) * b.n_layers + l) * (2 * b.n_kv * D);
    const float4 k = norm_rope(*reinterpret_cast<const float4*>(row + g * D + d0), b.eps, lane, reinterpret_cast<const float2*>(rope) + size_t(pos) * 32);
    const float4 v = *reinterpret_cast<const float4*>(row + (b.n_kv + g) * D + d0);
    const size_t at = ring_row(b, l, slot, g, pos) + d0;
    store_bf16x4(k_ring + at, k);
    store_bf16x4(v_ring + at, v);
}

// kernels.metal:1781-1812 `draft_embed`, one block of 256 threads per block row: row i of a slot's block sits at
// position lens[slot] + i; row 0 is the slot's next input (its bonus token) as rms_norm(embedding), the rows after it the
// mask embedding; `last` gets the normed context of the position before the block (zeros at position 0).
__global__ void embed_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ lens, const uint32_t* __restrict__ feed,
                             const float* __restrict__ mask_emb, const float* __restrict__ ctx_ring, const BlockDrafterDims b, uint32_t vocab, float* x, float* last,
                             uint32_t* meta) {
    pdl_start();
    __shared__ float red[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, slot = tin[2 * t], i = tin[2 * t + 1], len = lens[slot];
    uint32_t tok = feed[slot * FEED_W];
    if (tok >= vocab) tok = 0;  // (only a row of NaN logits can leave such an id in feed)
    if (tid == 0) {
        meta[2 * t] = slot;
        meta[2 * t + 1] = len + i;
    }
    const float* src = len ? ctx_ring + (size_t(slot) * b.ctx_ring_len + (len - 1) % b.ctx_ring_len) * b.hidden : nullptr;
    for (uint32_t d = tid; d < b.hidden; d += blockDim.x) last[size_t(t) * b.hidden + d] = src ? src[d] : 0.0f;
    if (i > 0) {
        for (uint32_t d = tid; d < b.hidden; d += blockDim.x) x[size_t(t) * b.hidden + d] = mask_emb[d];
        return;
    }
    const uint16_t* row = table + size_t(tok) * b.hidden;
    float ss = 0.0f;
    for (uint32_t d = tid; d < b.hidden; d += blockDim.x) { const float v = bf16_to_f32(row[d]); ss += v * v; }
    ss = warp_sum(ss);
    if (tid % 32 == 0) red[tid / 32] = ss;
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < blockDim.x / 32; w++) total += red[w];
    const float inv = 1.0f / sqrtf(total / float(b.hidden) + b.eps);
    for (uint32_t d = tid; d < b.hidden; d += blockDim.x) x[size_t(t) * b.hidden + d] = bf16_to_f32(row[d]) * inv;
}

// kernels.metal:1820-1840 `draft_conv` (tools/spec/drafter.py `Conv2`): out[t] = resid[t] (if any) + k0 x[t] + k1 x[t - 1]
// within a block, no predecessor for its row 0; the kernels are base [2][H] plus the row's corrections per 16 channels
// (k0's, then k1's; [rows][corr_stride], already times 1 / rms of the row). out must not be x.
__global__ void conv_kernel(const float* __restrict__ x, const float* __restrict__ corr, uint32_t corr_stride, const float* __restrict__ base,
                            const uint32_t* __restrict__ tin, const float* __restrict__ resid, uint32_t hidden, float* out) {
    pdl_start();
    const uint32_t t = blockIdx.x;
    const bool prev = tin[2 * t + 1] > 0;
    const float* c = corr + size_t(t) * corr_stride;
    for (uint32_t d = threadIdx.x; d < hidden; d += blockDim.x) {
        const size_t at = size_t(t) * hidden + d;
        float y = (base[d] + c[d / 16]) * x[at];
        if (prev) y += (base[hidden + d] + c[hidden / 16 + d / 16]) * x[at - hidden];
        out[at] = resid ? resid[at] + y : y;
    }
}

// The block rows' part of kernels.metal:749-801 `qkv_post` for a local layer: one block per row, a warp per head
// (query heads, then kv heads): q and k normed and turned in place, k and v rounded into the rings at the row's position.
__global__ void qkv_post_kernel(float* qkv, const uint32_t* __restrict__ meta, const float* __restrict__ rope, const BlockDrafterDims b, uint32_t layer,
                                uint16_t* k_ring, uint16_t* v_ring) {
    pdl_start();
    const uint32_t t = blockIdx.x, w = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], qw = (b.n_q + 2 * b.n_kv) * D;
    const float2* cs = reinterpret_cast<const float2*>(rope) + size_t(pos) * 32;
    float* head = qkv + size_t(t) * qw + w * D + d0;
    const float4 v = norm_rope(*reinterpret_cast<const float4*>(head), b.eps, lane, cs);
    *reinterpret_cast<float4*>(head) = v;
    if (w < b.n_q) return;
    const uint32_t g = w - b.n_q;
    const size_t at = ring_row(b, layer, slot, g, pos) + d0;
    store_bf16x4(k_ring + at, v);
    store_bf16x4(v_ring + at, *reinterpret_cast<const float4*>(qkv + size_t(t) * qw + (b.n_q + b.n_kv + g) * D + d0));
}

// A block row's attention (kernels.metal:891-1167 for a local layer, tools/spec/drafter.py `attend` + `block_mask`):
// grid (rows, query heads), four warps. The row at position p of the block that starts at p0 sees the ring's keys
// max(0, p - window) .. p0 - 1 and its block's rows p0 .. p0 + R - 1, all of them. A warp takes every fourth key: a
// lane holds four of the 128 dims of q, of the key and of its share of the output; online softmax per warp, the four
// merged through shared memory. Small (a block has at most 8 rows): nothing is tiled.
__global__ void attn_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ rows_of,
                            const uint16_t* __restrict__ k_ring, const uint16_t* __restrict__ v_ring, const BlockDrafterDims b,
                            uint32_t layer, float* out) {
    pdl_start();
    __shared__ float ms[4], ls[4];
    __shared__ float os[4][D];
    const uint32_t t = blockIdx.x, h = blockIdx.y, w = threadIdx.x / 32, lane = threadIdx.x % 32, d0 = 4 * lane;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], i = tin[2 * t + 1], rows = rows_of[t];
    const uint32_t p0 = pos - i, lo = pos > b.window ? pos - b.window : 0, hi = p0 + rows;  // kernels.metal:809 `key_lo`
    const uint32_t g = h / (b.n_q / b.n_kv), qw = (b.n_q + 2 * b.n_kv) * D;
    const float4 q = *reinterpret_cast<const float4*>(qkv + size_t(t) * qw + h * D + d0);
    float m = -INFINITY, l = 0.0f;
    float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t kp = lo + w; kp < hi; kp += 4) {
        const size_t at = ring_row(b, layer, slot, g, kp) + d0;
        const uint2 kb = *reinterpret_cast<const uint2*>(k_ring + at), vb = *reinterpret_cast<const uint2*>(v_ring + at);
        const float s = warp_sum(q.x * bf16lo(kb.x) + q.y * bf16hi(kb.x) + q.z * bf16lo(kb.y) + q.w * bf16hi(kb.y)) * b.scale;
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
    *reinterpret_cast<float4*>(out + (size_t(t) * b.n_q + h) * D + d0) = make_float4(oo.x / ll, oo.y / ll, oo.z / ll, oo.w / ll);
}

}  // namespace block

void launch_block_context(const float* kvp, const float* ctx, const float* ctx_inv, const uint32_t* meta, const uint32_t* on_path, const float* rope,
                          const BlockDrafterDims& b, uint32_t n, uint16_t* k_ring, uint16_t* v_ring, float* ctx_ring, cudaStream_t s) {
    launch_pdl(block::context_kernel, dim3(n, b.n_layers + 1), 32 * b.n_kv, 0, s, kvp, ctx, ctx_inv, meta, on_path, rope, b, k_ring, v_ring, ctx_ring);
}
void launch_block_embed(const uint16_t* table, const uint32_t* tin, const uint32_t* lens, const uint32_t* feed, const float* mask_emb, const float* ctx_ring,
                        const BlockDrafterDims& b, uint32_t vocab, uint32_t rows, float* x, float* last, uint32_t* meta, cudaStream_t s) {
    launch_pdl(block::embed_kernel, rows, 256, 0, s, table, tin, lens, feed, mask_emb, ctx_ring, b, vocab, x, last, meta);
}
void launch_block_conv(const float* x, const float* corr, uint32_t corr_stride, const float* base, const uint32_t* tin, const float* resid, uint32_t hidden,
                       uint32_t rows, float* out, cudaStream_t s) {
    launch_pdl(block::conv_kernel, rows, 256, 0, s, x, corr, corr_stride, base, tin, resid, hidden, out);
}
void launch_block_qkv_post(float* qkv, const uint32_t* meta, const float* rope, const BlockDrafterDims& b, uint32_t layer, uint32_t rows, uint16_t* k_ring,
                           uint16_t* v_ring, cudaStream_t s) {
    launch_pdl(block::qkv_post_kernel, rows, 32 * (b.n_q + b.n_kv), 0, s, qkv, meta, rope, b, layer, k_ring, v_ring);
}
void launch_block_attn(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* rows_of, const uint16_t* k_ring,
                       const uint16_t* v_ring, const BlockDrafterDims& b, uint32_t layer, uint32_t rows, float* out, cudaStream_t s) {
    launch_pdl(block::attn_kernel, dim3(rows, b.n_q), 128, 0, s, qkv, meta, tin, rows_of, k_ring, v_ring, b, layer, out);
}

}  // namespace vlt
