// TEST INFRASTRUCTURE (CPU oracle, parity unpinned: see limite.hpp). The forward pass of the reference's own
// architecture, statement for statement from the engine's dispatch order (engine/src/engine/encode.rs:99-192,383-394) and
// its kernels (engine/src/kernels.metal): `embed` :82-114, the matmul epilogues :184-209, `qkv_post` / `new_key`
// :725-801,910-945 (q/k norm, RoPE on local layers, value embeddings, cache writes, XSA directions, attention gates),
// the attention's visibility :809-811,1019-1062, `attn_dec_reduce` :1314-1362 (XSA, gate), `mudd` :1364-1407.
// Included by model.hpp after `Engine`. As everywhere in this oracle a matmul's input activations are rounded to bf16
// and the softmax subtracts the row maximum (the reference's scores are bounded by its q/k norms and it does not).
#pragma once
#include <algorithm>
#include <cmath>
#include <vector>

namespace orc {

namespace limite {

inline float sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }
// kernels.metal:31-38: erf by Abramowitz & Stegun 7.1.26, and gelu over it.
inline float erf_f(float x) {
    const float a = std::fabs(x), t = 1.0f / (1.0f + 0.3275911f * a);
    const float y = 1.0f - (((((1.061405429f * t - 1.453152027f) * t) + 1.421413741f) * t - 0.284496736f) * t + 0.254829592f) * t * std::exp(-a * a);
    return std::copysign(y, x);
}
inline float gelu(float x) { return 0.5f * x * (1.0f + erf_f(x * 0.70710678118654752f)); }

// kernels.metal:727-736 `norm_rope` on a head of 128: rms_norm, then (if `rope`) 32 interleaved pairs of dims 0..63 turn.
inline void norm_rope(float* h, bool rope, uint32_t pos, float eps, const std::vector<float>& freq) {
    float ss = 0.0f;
    for (uint32_t d = 0; d < Limite::D; d++) ss += h[d] * h[d];
    const float inv = 1.0f / std::sqrt(ss / float(Limite::D) + eps);
    for (uint32_t d = 0; d < Limite::D; d++) h[d] *= inv;
    if (!rope) return;
    for (uint32_t j = 0; j < 32; j++) {
        float c, s;
        rope_cs(pos, freq[j], c, s);
        const float a0 = h[2 * j], a1 = h[2 * j + 1];
        h[2 * j] = c * a0 + s * a1;
        h[2 * j + 1] = c * a1 - s * a0;
    }
}

}  // namespace limite

inline void limite_forward(Engine& e, const Plan& p) {
    using namespace limite;
    const ModelDesc& md = e.md;
    Limite& lm = *e.lim;
    const uint32_t n = p.n, H = md.d, D = Limite::D, NQ = md.n_heads, NKV = md.n_kv, G = NQ / NKV, QW = md.qkv_w(), FFN = md.ffn;
    const uint32_t koff = NQ * D, voff = koff + NKV * D;
    // embed, kernels.metal:82-114: a GPU-fed token resolved in place; out = rms_norm(embedding).
    e.meta.assign(2 * n, 0);
    std::vector<float> hist0(size_t(n) * H), hist12, hist23, hmain(size_t(n) * H);
    for (uint32_t t = 0; t < n; t++) {
        const uint32_t slot = e.tin[2 * t];
        uint32_t tok = e.tokens[t], depth = e.tin[2 * t + 1];
        if (tok >= FEED_ROW) {
            const uint32_t i = tok - FEED_ROW, node = e.tree[slot * FEED_W + i];
            tok = e.feed[slot * FEED_W + i];
            depth = node_depth(node);
            e.vis[t] = node_sees(node);
        }
        e.tokens[t] = tok;
        e.meta[2 * t] = slot;
        e.meta[2 * t + 1] = e.lens[slot] + depth;
        float ss = 0.0f;
        for (uint32_t i = 0; i < H; i++) { const float v = bf16_to_f32(e.embed[size_t(tok) * H + i]); hist0[size_t(t) * H + i] = v; ss += v * v; }
        const float inv = 1.0f / std::sqrt(ss / float(H) + md.eps);
        for (uint32_t i = 0; i < H; i++) hist0[size_t(t) * H + i] *= inv;
    }
    e.taps_all.assign(e.tap_layers.size() * size_t(n) * H, 0.0f);
    std::vector<float> xattn(size_t(n) * H), base(size_t(n) * H), inv(n), qkv(size_t(n) * QW), acc(size_t(n) * std::max<size_t>({size_t(QW), size_t(2) * FFN, size_t(H)})),
        attn(size_t(n) * H), mixed(size_t(n) * H), act(size_t(n) * FFN), vdir(size_t(n) * NKV * D), gates(size_t(n) * NQ);
    const std::vector<float>* cur = &hist0;  // encode.rs:107-114 `resid_in`
    for (uint32_t li = 0; li < md.n_layers; li++) {
        const Layer& L = e.layers[li];
        const LimiteLayer& X = lm.layers[li];
        const float* h = cur->data();
        const float* x = h;   // the attention's input
        const float* bs = h;  // the residual base
        const int site = Limite::mudd_site(li);
        if (site >= 0) {  // kernels.metal:1364-1407 `mudd`
            const std::vector<float>& tap1 = site == 0 ? hist12 : hist23;
            const float* mix = lm.mudd_mix + size_t(site) * 2 * 3 * 33;
            for (uint32_t t = 0; t < n; t++) {
                const float* c = h + size_t(t) * H;
                float ss = 0.0f;
                for (uint32_t i = 0; i < H; i++) ss += c[i] * c[i];
                const float iv = 1.0f / std::sqrt(ss / float(H) + md.eps);
                float inner[32], w[6];
                for (uint32_t j = 0; j < 32; j++) {
                    float s = 0.0f;
                    for (uint32_t k = 0; k < H; k++) s += c[k] * iv * lm.mudd_dense1[size_t(j) * H + k];
                    inner[j] = gelu(s);
                }
                for (uint32_t r = 0; r < 6; r++) {
                    float s = 0.0f;
                    for (uint32_t j = 0; j < 32; j++) s += inner[j] * mix[r * 33 + j];
                    w[r] = s + mix[r * 33 + 32];
                }
                for (uint32_t i = 0; i < H; i++) {
                    const size_t o = size_t(t) * H + i;
                    const float a = hist0[o], b = tap1[o], xc = c[i];
                    xattn[o] = w[0] * a + w[1] * b + w[2] * xc;
                    base[o] = w[3] * a + w[4] * b + w[5] * xc;
                }
            }
            x = xattn.data();
            bs = base.data();
        }
        // qkv = (W x) / rms(x) * qkv_scale (EPI_NORM, kernels.metal:188).
        inv_rms(x, n, H, md.eps, inv.data());
        matmul_raw(L.qkv, x, n, acc.data());
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t j = 0; j < QW; j++) qkv[size_t(t) * QW + j] = acc[size_t(t) * QW + j] * inv[t] * X.qkv_scale;
        // qkv_post / new_key: q and k normed (turned on local layers), value embeddings, K/V into the cache at the row's
        // cache position, XSA directions, attention gates.
        for (uint32_t t = 0; t < n; t++) {
            const uint32_t slot = e.meta[2 * t], pos = e.meta[2 * t + 1], row = e.tin[2 * t + 1];
            const uint32_t cpos = e.meta[2 * (t - row) + 1] + row;  // kernels.metal:74-77 `cache_pos`
            float* qr = qkv.data() + size_t(t) * QW;
            const float* xt = x + size_t(t) * H;
            for (uint32_t hq = 0; hq < NQ; hq++) {
                norm_rope(qr + hq * D, !X.global, pos, md.eps, e.rope_freq);
                float s = 0.0f;  // 2 sigmoid(rms_norm(x)[:128] . attn_gate[h]), kernels.metal:781-784
                for (uint32_t d = 0; d < D; d++) s += xt[d] * inv[t] * X.attn_gate[hq * D + d];
                gates[size_t(t) * NQ + hq] = 2.0f * sigmoid(s);
            }
            for (uint32_t g = 0; g < NKV; g++) {
                float* k = qr + koff + g * D;
                float* v = qr + voff + g * D;
                norm_rope(k, !X.global, pos, md.eps, e.rope_freq);
                if (X.ve_gate) {  // kernels.metal:738-747 `add_ve`
                    float s = 0.0f;
                    for (uint32_t d = 0; d < 12; d++) s += xt[d] * inv[t] * X.ve_gate[g * 12 + d];
                    const float gate = 2.0f * sigmoid(s);
                    const uint16_t* ve = lm.value_embed + size_t(e.tokens[t]) * NKV * D + g * D;
                    for (uint32_t d = 0; d < D; d++) v[d] += gate * bf16_to_f32(ve[d]);
                }
                uint16_t* kc = X.global ? e.k_cache.data() + e.kv_row(X.kv_index, slot, g, cpos) : lm.k_local.data() + e.limite_ring_row(X.kv_index, slot, g, cpos);
                uint16_t* vc = X.global ? e.v_cache.data() + e.kv_row(X.kv_index, slot, g, cpos) : lm.v_local.data() + e.limite_ring_row(X.kv_index, slot, g, cpos);
                float nrm = 0.0f;
                for (uint32_t d = 0; d < D; d++) { kc[d] = f32_to_bf16(k[d]); vc[d] = f32_to_bf16(v[d]); nrm += v[d] * v[d]; }
                nrm = std::max(std::sqrt(nrm), Limite::XSA_EPS);
                for (uint32_t d = 0; d < D; d++) vdir[(size_t(t) * NKV + g) * D + d] = v[d] / nrm;
            }
        }
        // Attention per tile: cached keys below the tile's first position that the row's window reaches (a global layer's
        // window is everything), the tile's own rows under `vis`; then XSA and the gate (`attn_dec_reduce`).
        const float sl = md.attn_scale;
#pragma omp parallel for schedule(dynamic) collapse(2)
        for (int64_t ti = 0; ti < int64_t(p.n_tiles); ti++)
            for (int64_t hq = 0; hq < int64_t(NQ); hq++) {
                const uint32_t t0 = e.tiles[2 * ti], T = e.tiles[2 * ti + 1], g = uint32_t(hq) / G;
                const uint32_t slot = e.meta[2 * t0], p0 = e.meta[2 * t0 + 1];
                for (uint32_t i = 0; i < T; i++) {
                    const uint32_t t = t0 + i, pos = e.meta[2 * t + 1];
                    const uint32_t lo = X.global ? 0u : (pos > Limite::WINDOW ? pos - Limite::WINDOW : 0u);  // kernels.metal:809 `key_lo`
                    const float* q = qkv.data() + size_t(t) * QW + hq * D;
                    std::vector<float> sc;
                    std::vector<uint32_t> keys;
                    for (uint32_t kp = lo; kp < p0 + T; kp++) {
                        const bool seen = kp < p0 || ((e.vis[t] >> (kp - p0)) & 1u);
                        if (seen) keys.push_back(kp);
                    }
                    float mx = -INFINITY;
                    for (uint32_t kp : keys) {
                        const uint16_t* kr = X.global ? e.k_cache.data() + e.kv_row(X.kv_index, slot, g, kp) : lm.k_local.data() + e.limite_ring_row(X.kv_index, slot, g, kp);
                        float a = 0.0f;
                        for (uint32_t d = 0; d < D; d++) a += q[d] * bf16_to_f32(kr[d]);
                        sc.push_back(a * sl);
                        mx = std::max(mx, sc.back());
                    }
                    float l = 0.0f, o[Limite::D] = {};
                    for (size_t k = 0; k < keys.size(); k++) {
                        const float pz = std::exp(sc[k] - mx);
                        l += pz;
                        const uint16_t* vr = X.global ? e.v_cache.data() + e.kv_row(X.kv_index, slot, g, keys[k]) : lm.v_local.data() + e.limite_ring_row(X.kv_index, slot, g, keys[k]);
                        for (uint32_t d = 0; d < D; d++) o[d] += pz * bf16_to_f32(vr[d]);
                    }
                    const float* vd = vdir.data() + (size_t(t) * NKV + g) * D;
                    float pr = 0.0f;
                    for (uint32_t d = 0; d < D; d++) { o[d] /= l; pr += o[d] * vd[d]; }
                    for (uint32_t d = 0; d < D; d++) attn[size_t(t) * H + hq * D + d] = (o[d] - X.xsa[hq] * pr * vd[d]) * gates[size_t(t) * NQ + hq];
                }
            }
        // mixed = resid_attn * base + post_attn * (o_scale * W_o attn)   (EPI_RESID, kernels.metal:190-195)
        matmul_raw(L.o, attn.data(), n, acc.data());
        for (size_t i = 0; i < size_t(n) * H; i++) mixed[i] = X.resid_attn * bs[i] + X.post_attn * (X.o_scale * acc[i]);
        inv_rms(mixed.data(), n, H, md.eps, inv.data());
        matmul_raw(L.gate_up, mixed.data(), n, acc.data());
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t j = 0; j < FFN; j++) {  // kernels.metal:204-209
                const float gt = acc[size_t(t) * 2 * FFN + 2 * j] * inv[t], up = acc[size_t(t) * 2 * FFN + 2 * j + 1] * inv[t];
                act[size_t(t) * FFN + j] = gt * sigmoid(gt) * up;
            }
        matmul_raw(L.down, act.data(), n, acc.data());
        std::vector<float>& out = li == 11 ? hist12 : li == 22 ? hist23 : hmain;  // encode.rs:116-122 `resid_out`
        out.resize(size_t(n) * H);
        for (size_t i = 0; i < size_t(n) * H; i++) out[i] = X.resid_mlp * mixed[i] + X.post_mlp * acc[i];
        cur = &out;
        for (size_t k = 0; k < e.tap_layers.size(); k++) {  // kernels.metal:133-148 `tap_rows`
            if (e.tap_layers[k] != li) continue;
            std::vector<float> tinv(n);
            inv_rms(out.data(), n, H, md.eps, tinv.data());
            for (uint32_t t = 0; t < n; t++)
                for (uint32_t i = 0; i < H; i++) e.taps_all[(k * n + t) * H + i] = round_bf16(out[size_t(t) * H + i] * tinv[t]);
        }
    }
    // encode.rs:383-394: final norm of the hidden and head rows, the head with the cap, padding ids masked.
    const float* hf = cur->data();
    inv_rms(hf, n, H, md.eps, inv.data());
    e.taps.resize(size_t(n) * H);
    for (uint32_t t = 0; t < n; t++)
        for (uint32_t i = 0; i < H; i++) e.taps[size_t(t) * H + i] = round_bf16(hf[size_t(t) * H + i] * inv[t]);
    e.hidden_out.resize(size_t(p.n_hidden) * H);
    for (uint32_t r = 0; r < p.n_hidden; r++)
        for (uint32_t i = 0; i < H; i++) e.hidden_out[size_t(r) * H + i] = hf[size_t(e.hidden_rows[r]) * H + i] * inv[e.hidden_rows[r]];
    e.out_ids.assign(p.n_head, 0);
    if (p.n_head) {
        std::vector<float> hx(size_t(p.n_head) * H);
        for (uint32_t r = 0; r < p.n_head; r++)
            for (uint32_t i = 0; i < H; i++) hx[size_t(r) * H + i] = hf[size_t(e.head_rows[r]) * H + i] * inv[e.head_rows[r]];
        e.logits.resize(size_t(p.n_head) * md.vocab);
        matmul_raw(e.head, hx.data(), p.n_head, e.logits.data());
        for (uint32_t r = 0; r < p.n_head; r++)
            for (uint32_t j = 0; j < md.vocab; j++) {
                float& l = e.logits[size_t(r) * md.vocab + j];
                l = j < md.vocab_real ? 23.0f * sigmoid((l + 5.0f) / 7.5f) : -INFINITY;  // kernels.metal:196-199
            }
    }
    e.finish_step(p);
}

}  // namespace orc
