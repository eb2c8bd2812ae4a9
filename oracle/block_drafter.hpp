// TEST INFRASTRUCTURE: a CPU restatement of the reference's block drafter, used only as the checker.
//
// The model is tools/spec/drafter.py (`Drafter`, `Layer`, `Conv2`, `attend`, `block_mask`); the way it runs in the
// engine -- the context's keys and values in rings per (layer, slot), the normed context in a ring per slot, the block
// rows' inputs, the convolutions' corrections through a matmul, raw logits, draft_top and draft_tree behind them --
// is engine/src/engine/drafter.rs:278-447 with the kernels of kernels.metal:1726-1840 (`draft_kv`, `draft_ctx`,
// `draft_embed`, `draft_conv`) and the local-layer attention conventions of kernels.metal:704-736,808-811 (`norm_rope`,
// `key_lo`). The file is what tools/spec/export.py writes.
//
// Parity: pinned. tests/test_block_drafter_oracle.py holds this file to outputs of the unmodified Python model
// (tests/golden/block_drafter.npz, made by tests/golden/make_block_drafter_golden.py).
//
// Conventions that differ from the reference's, as everywhere in this oracle: a matmul's input activations are rounded
// to bf16 (the product's kernels take them so); the softmax subtracts the row maximum. The reference's shapes are
// constants (hidden 1280, 10 query and 2 kv heads of 128, FFN 3328); here the hidden width and the FFN come from the
// file and heads stay 128 wide.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "linear.hpp"

namespace orc {

struct BlockDrafter {
    static constexpr uint32_t D = 128, CONV_KC = 192, CANDS = 4;
    VltFile file;
    uint32_t n_layers = 0, n_taps = 0, block = 0, window = 0, v = 0, H = 0, NQ = 0, NKV = 0, FFN = 0;
    std::vector<uint32_t> taps, vocab;
    std::vector<Matrix> fc;
    Matrix kv_all, inject, head;
    const float* mask_emb = nullptr;
    struct DLayer {
        Matrix qkv, o, gate_up, down;
        const float* conv_base[4];
        Matrix conv_corr[4];
    };
    std::vector<DLayer> layers;
    // What the engine it runs in supplies (drafter.rs uses the engine's globals): epsilon, attention scale, RoPE table.
    float eps = 0.0f, scale = 0.0f;
    std::vector<float> rope_freq;  // 32 pairs: the first 64 of a head's 128 dims turn
    // State: rings per (layer, slot) of bf16 keys and values, a ring per slot of the normed context.
    uint32_t max_seqs = 0, ring = 0, ctx_ring_len = 0;
    std::vector<uint16_t> k_ring, v_ring;  // [layer][slot][NKV][ring][D]
    std::vector<float> ctx_ring;           // [slot][ctx_ring_len][H]
    // The last block pass: final normed rows [rows][H], raw logits [rows][v], candidates.
    std::vector<float> hfin, logits, cand_q;
    std::vector<uint32_t> cand;

    static bool is_block_drafter(const VltFile& f) { return f.has("kv_all"); }

    BlockDrafter(const std::string& path, float eps_, float scale_, const std::vector<float>& freq) : file(VltFile::load(path)), eps(eps_), scale(scale_), rope_freq(freq) {
        const std::vector<float> m = file.f32s("meta");
        if (m.size() < 5 || m.size() != 5 + size_t(m[1])) throw std::runtime_error(path + ": meta is not a block drafter's");
        n_layers = uint32_t(m[0]); n_taps = uint32_t(m[1]); block = uint32_t(m[2]); window = uint32_t(m[3]); v = uint32_t(m[4]);
        for (uint32_t k = 0; k < n_taps; k++) taps.push_back(uint32_t(m[5 + k]));
        if (rope_freq.size() != 32) throw std::runtime_error("the block drafter turns 32 pairs: the engine's RoPE table must have 32 frequencies");
        H = file.tensor("fc.0").shape.at(1);
        NQ = H / D;
        const uint32_t kv_rows = file.tensor("kv_all").shape.at(0);
        NKV = kv_rows / (n_layers * 2 * D);
        FFN = file.tensor("D00.down").shape.at(1);
        for (uint32_t k = 0; k < n_taps; k++) fc.push_back(load_matrix(file, "fc." + std::to_string(k), H, H));
        kv_all = load_matrix(file, "kv_all", n_layers * 2 * NKV * D, H);
        inject = load_matrix(file, "inject", H, H);
        head = load_matrix(file, "head", v, H);
        mask_emb = reinterpret_cast<const float*>(file.ptr(file.get("mask_emb", F32, {H})));
        for (uint32_t i = 0; i < n_layers; i++) {
            char nm[48];
            auto name = [&](const char* k) { std::snprintf(nm, sizeof nm, "D%02u.%s", i, k); return std::string(nm); };
            DLayer l;
            l.qkv = load_matrix(file, name("qkv"), (NQ + 2 * NKV) * D, H);
            l.o = load_matrix(file, name("o"), H, NQ * D);
            l.gate_up = load_matrix(file, name("gate_up"), 2 * FFN, H);
            l.down = load_matrix(file, name("down"), H, FFN);
            for (uint32_t c = 0; c < 4; c++) {
                const std::string cn = "conv" + std::to_string(c);
                l.conv_base[c] = reinterpret_cast<const float*>(file.ptr(file.get(name((cn + ".base").c_str()), F32, {2, H})));
                l.conv_corr[c] = load_matrix(file, name((cn + ".corr").c_str()), CONV_KC, H);
            }
            layers.push_back(l);
        }
        for (float id : file.f32s("vocab")) vocab.push_back(uint32_t(id));
        if (vocab.size() != v) throw std::runtime_error(path + ": vocab has " + std::to_string(vocab.size()) + " ids for a head of " + std::to_string(v));
    }

    // drafter.rs:175-184: rings of window + max_chunk positions, the context ring of max_chunk.
    void init_state(uint32_t seqs, uint32_t max_chunk) {
        max_seqs = seqs;
        ring = window + max_chunk;
        ctx_ring_len = max_chunk;
        k_ring.assign(size_t(n_layers) * seqs * NKV * ring * D, 0);
        v_ring.assign(k_ring.size(), 0);
        ctx_ring.assign(size_t(seqs) * ctx_ring_len * H, 0.0f);
    }
    size_t ring_row(uint32_t layer, uint32_t slot, uint32_t g, uint32_t pos) const {  // kernels.metal:710 `kv_row_of`, local
        return ((size_t(layer) * max_seqs + slot) * NKV + g) * ring * D + size_t(pos % ring) * D;
    }

    // kernels.metal:727-736 `norm_rope`: rms_norm over the head, then RoPE on dims 0..63 as 32 interleaved pairs.
    void norm_rope(float* h, uint32_t pos) const {
        float ss = 0.0f;
        for (uint32_t d = 0; d < D; d++) ss += h[d] * h[d];
        const float inv = 1.0f / std::sqrt(ss / float(D) + eps);
        for (uint32_t d = 0; d < D; d++) h[d] *= inv;
        for (uint32_t j = 0; j < 32; j++) {
            float c, s;
            rope_cs(pos, rope_freq[j], c, s);
            const float a0 = h[2 * j], a1 = h[2 * j + 1];
            h[2 * j] = c * a0 + s * a1;
            h[2 * j + 1] = c * a1 - s * a0;
        }
    }

    // drafter.rs:283-311 step 1 and kernels.metal:1735-1774: the fused context of n tokens (tap k of token t at
    // tap_rows[k] + t * H, bf16 values), its keys and values into the rings and its normed rows into the context ring,
    // for the tokens on_path (NULL: all of them).
    void context(uint32_t n, const std::vector<const float*>& tap_rows, const uint32_t* meta, const uint32_t* on_path) {
        std::vector<float> ctx(size_t(n) * H, 0.0f), acc(size_t(n) * std::max<size_t>(H, kv_all.m)), inv(n);
        for (uint32_t k = 0; k < n_taps; k++) {
            matmul_raw(fc[k], tap_rows[k], n, acc.data());
            for (size_t i = 0; i < size_t(n) * H; i++) ctx[i] += acc[i];
        }
        inv_rms(ctx.data(), n, H, eps, inv.data());
        matmul_raw(kv_all, ctx.data(), n, acc.data());
        const uint32_t W = kv_all.m;
        for (uint32_t t = 0; t < n; t++) {
            if (on_path && !on_path[t]) continue;
            const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1];
            for (uint32_t l = 0; l < n_layers; l++)
                for (uint32_t g = 0; g < NKV; g++) {
                    float k[D], vv[D];
                    for (uint32_t d = 0; d < D; d++) {
                        k[d] = acc[size_t(t) * W + (l * 2 * NKV + g) * D + d] * inv[t];
                        vv[d] = acc[size_t(t) * W + (l * 2 * NKV + NKV + g) * D + d] * inv[t];
                    }
                    norm_rope(k, pos);
                    const size_t at = ring_row(l, slot, g, pos);
                    for (uint32_t d = 0; d < D; d++) { k_ring[at + d] = f32_to_bf16(k[d]); v_ring[at + d] = f32_to_bf16(vv[d]); }
                }
            float* dst = ctx_ring.data() + (size_t(slot) * ctx_ring_len + pos % ctx_ring_len) * H;
            for (uint32_t d = 0; d < H; d++) dst[d] = ctx[size_t(t) * H + d] * inv[t];
        }
    }

    // kernels.metal:1820-1840 `draft_conv` behind its corrections' matmul (drafter.rs:356-368).
    void conv(const DLayer& L, uint32_t c, const float* x, const uint32_t* row_in_block, uint32_t rows, const float* resid, float* out) const {
        std::vector<float> corr(size_t(rows) * CONV_KC), inv(rows);
        inv_rms(x, rows, H, eps, inv.data());
        matmul_raw(L.conv_corr[c], x, rows, corr.data());
        const float* base = L.conv_base[c];
        for (uint32_t t = 0; t < rows; t++)
            for (uint32_t d = 0; d < H; d++) {
                const float* cr = corr.data() + size_t(t) * CONV_KC;
                float y = (base[d] + cr[d / 16] * inv[t]) * x[size_t(t) * H + d];
                if (row_in_block[t] > 0) y += (base[H + d] + cr[H / 16 + d / 16] * inv[t]) * x[size_t(t - 1) * H + d];
                out[size_t(t) * H + d] = resid ? resid[size_t(t) * H + d] + y : y;
            }
    }

    struct Block { uint32_t slot, rows, p0; const uint16_t* bonus_row; };  // p0: the bonus token's position; its embedding row (bf16)

    // drafter.rs:312-447 steps 2 and 3 without the tree: the blocks' rows through the layers; leaves hfin and logits.
    void blocks(const std::vector<Block>& bl) {
        uint32_t rows = 0;
        for (const Block& b : bl) rows += b.rows;
        std::vector<float> x(size_t(rows) * H), last(size_t(rows) * H), acc(size_t(rows) * std::max<size_t>({size_t(H), size_t(2) * FFN, size_t(NQ + 2 * NKV) * D}));
        std::vector<uint32_t> slot_of(rows), row_in(rows), pos_of(rows), p0_of(rows), rows_of(rows);
        uint32_t t = 0;
        for (const Block& b : bl)
            for (uint32_t i = 0; i < b.rows; i++, t++) {
                slot_of[t] = b.slot; row_in[t] = i; pos_of[t] = b.p0 + i; p0_of[t] = b.p0; rows_of[t] = b.rows;
                float* xr = x.data() + size_t(t) * H;
                if (i == 0) {  // kernels.metal:1805-1811: rms_norm(embedding)
                    float ss = 0.0f;
                    for (uint32_t d = 0; d < H; d++) { xr[d] = bf16_to_f32(b.bonus_row[d]); ss += xr[d] * xr[d]; }
                    const float inv = 1.0f / std::sqrt(ss / float(H) + eps);
                    for (uint32_t d = 0; d < H; d++) xr[d] *= inv;
                } else {
                    std::copy_n(mask_emb, H, xr);
                }
                // The normed context of the position before the block (zeros before any: a block at position 0 has none).
                const float* src = b.p0 ? ctx_ring.data() + (size_t(b.slot) * ctx_ring_len + (b.p0 - 1) % ctx_ring_len) * H : nullptr;
                for (uint32_t d = 0; d < H; d++) last[size_t(t) * H + d] = src ? src[d] : 0.0f;
            }
        matmul_raw(inject, last.data(), rows, acc.data());
        for (size_t i = 0; i < size_t(rows) * H; i++) x[i] += acc[i];

        const uint32_t QW = (NQ + 2 * NKV) * D, G = NQ / NKV;
        std::vector<float> cx(size_t(rows) * H), co(size_t(rows) * H), mixed(size_t(rows) * H), attn(size_t(rows) * NQ * D), inv(rows), act(size_t(rows) * FFN);
        for (uint32_t li = 0; li < n_layers; li++) {
            const DLayer& L = layers[li];
            conv(L, 0, x.data(), row_in.data(), rows, nullptr, cx.data());
            inv_rms(cx.data(), rows, H, eps, inv.data());
            matmul_raw(L.qkv, cx.data(), rows, acc.data());
            std::vector<float> qkv(acc.begin(), acc.begin() + size_t(rows) * QW);
            // q and k normed and turned; the rows' K/V into the rings (bf16) before any row attends: a row sees its whole block.
            for (uint32_t r = 0; r < rows; r++) {
                float* row = qkv.data() + size_t(r) * QW;
                for (uint32_t j = 0; j < QW; j++) row[j] *= inv[r];
                for (uint32_t h = 0; h < NQ + NKV; h++) norm_rope(row + h * D, pos_of[r]);
                for (uint32_t g = 0; g < NKV; g++) {
                    const size_t at = ring_row(li, slot_of[r], g, pos_of[r]);
                    for (uint32_t d = 0; d < D; d++) {
                        k_ring[at + d] = f32_to_bf16(row[(NQ + g) * D + d]);
                        v_ring[at + d] = f32_to_bf16(row[(NQ + NKV + g) * D + d]);
                    }
                }
            }
            for (uint32_t r = 0; r < rows; r++) {
                const uint32_t pos = pos_of[r], p0 = p0_of[r], lo = pos > window ? pos - window : 0;  // kernels.metal:809 `key_lo`
                for (uint32_t h = 0; h < NQ; h++) {
                    const float* q = qkv.data() + size_t(r) * QW + h * D;
                    const uint32_t g = h / G;
                    std::vector<float> sc;
                    std::vector<uint32_t> keys;
                    for (uint32_t kp = lo; kp < p0 + rows_of[r]; kp++) keys.push_back(kp);  // the context below the block, then the block
                    float mx = -INFINITY;
                    for (uint32_t kp : keys) {
                        const uint16_t* kr = k_ring.data() + ring_row(li, slot_of[r], g, kp);
                        float a = 0.0f;
                        for (uint32_t d = 0; d < D; d++) a += q[d] * bf16_to_f32(kr[d]);
                        sc.push_back(a * scale);
                        mx = std::max(mx, sc.back());
                    }
                    float l = 0.0f, o[D] = {};
                    for (size_t i = 0; i < keys.size(); i++) {
                        const float p = std::exp(sc[i] - mx);
                        l += p;
                        const uint16_t* vr = v_ring.data() + ring_row(li, slot_of[r], g, keys[i]);
                        for (uint32_t d = 0; d < D; d++) o[d] += p * bf16_to_f32(vr[d]);
                    }
                    for (uint32_t d = 0; d < D; d++) attn[(size_t(r) * NQ + h) * D + d] = o[d] / l;
                }
            }
            matmul_raw(L.o, attn.data(), rows, co.data());
            conv(L, 1, co.data(), row_in.data(), rows, x.data(), mixed.data());
            conv(L, 2, mixed.data(), row_in.data(), rows, nullptr, cx.data());
            inv_rms(cx.data(), rows, H, eps, inv.data());
            matmul_raw(L.gate_up, cx.data(), rows, acc.data());
            for (uint32_t r = 0; r < rows; r++)
                for (uint32_t j = 0; j < FFN; j++) {  // kernels.metal:204-209
                    const float gt = acc[size_t(r) * 2 * FFN + 2 * j] * inv[r], up = acc[size_t(r) * 2 * FFN + 2 * j + 1] * inv[r];
                    act[size_t(r) * FFN + j] = gt * (1.0f / (1.0f + std::exp(-gt))) * up;
                }
            matmul_raw(L.down, act.data(), rows, co.data());
            conv(L, 3, co.data(), row_in.data(), rows, mixed.data(), x.data());
        }
        hfin.assign(size_t(rows) * H, 0.0f);
        inv_rms(x.data(), rows, H, eps, inv.data());
        for (uint32_t r = 0; r < rows; r++)
            for (uint32_t d = 0; d < H; d++) hfin[size_t(r) * H + d] = x[size_t(r) * H + d] * inv[r];
        logits.assign(size_t(rows) * v, 0.0f);
        matmul_raw(head, hfin.data(), rows, logits.data());
    }
};

}  // namespace orc
