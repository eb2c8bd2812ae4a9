// CPU oracle (test infrastructure only): what the engine's step and the drafters share -- a model's shape, a weight
// matrix (bf16, or int8 with bf16 scales per group of consecutive k: kernels.metal:150-181) and the matmul, RoPE and
// RMS helpers on host memory. See model.hpp for the conventions.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "bits.hpp"
#include "vlt.hpp"

namespace orc {

struct ModelDesc {
    uint32_t n_layers, d, n_heads, n_kv, hd, ffn, vocab, vocab_real;
    float eps;
    uint32_t page;
    float attn_scale;
    uint32_t qkv_w() const { return (n_heads + 2 * n_kv) * hd; }
};

struct Matrix {
    const uint8_t* w = nullptr;
    const uint16_t* scales = nullptr;  // int8 only: [m][k / group]
    uint32_t m = 0, k = 0, group = 0;
    bool int8 = false;
};

// engine/src/model.rs:81-103 `matrix`: bf16, or int8 with `<name>.scale`. The reference accepts
// groups of 8..256; a whole row per scale (group = k) is accepted here as well.
inline Matrix load_matrix(const VltFile& f, const std::string& name, uint32_t m, uint32_t k) {
    const Tensor& t = f.tensor(name);
    Matrix out;
    out.m = m;
    out.k = k;
    if (t.dtype != I8) {
        out.w = f.ptr(f.get(name, BF16, {m, k}));
        return out;
    }
    out.w = f.ptr(f.get(name, I8, {m, k}));
    const Tensor& s = f.tensor(name + ".scale");
    const uint32_t groups = s.shape.size() > 1 ? s.shape[1] : 0;
    const uint32_t group = k / std::max(groups, 1u);
    if (group < 8 || (groups > 1 && (group & (group - 1))) || group * groups != k) throw std::runtime_error(name + ".scale: bad group count");
    out.scales = reinterpret_cast<const uint16_t*>(f.ptr(f.get(name + ".scale", BF16, {m, groups})));
    out.group = group;
    out.int8 = true;
    return out;
}

// acc[t][row] = sum_k W[row][k] * bf16(X[t][k]), int8 groups scaled as they are added.
inline void matmul_raw(const Matrix& W, const float* X, uint32_t n, float* acc) {
    std::vector<float> xb(size_t(n) * W.k);
    for (size_t i = 0; i < xb.size(); i++) xb[i] = round_bf16(X[i]);
#pragma omp parallel
    {
        std::vector<float> wr(W.k);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < int64_t(W.m); r++) {
            if (W.int8) {
                const int8_t* q = reinterpret_cast<const int8_t*>(W.w) + uint64_t(r) * W.k;
                for (uint32_t i = 0; i < W.k; i++) wr[i] = float(q[i]);
            } else {
                const uint16_t* b = reinterpret_cast<const uint16_t*>(W.w) + uint64_t(r) * W.k;
                for (uint32_t i = 0; i < W.k; i++) wr[i] = bf16_to_f32(b[i]);
            }
            const uint32_t group = W.int8 ? W.group : W.k, ng = W.k / group;
            for (uint32_t t = 0; t < n; t++) {
                const float* x = xb.data() + size_t(t) * W.k;
                float total = 0.0f;
                for (uint32_t g = 0; g < ng; g++) {
                    float a = 0.0f;
#pragma omp simd reduction(+ : a)
                    for (uint32_t i = g * group; i < (g + 1) * group; i++) a += wr[i] * x[i];
                    total += W.int8 ? a * bf16_to_f32(W.scales[uint64_t(r) * ng + g]) : a;
                }
                acc[size_t(t) * W.m + r] = total;
            }
        }
    }
}

// engine.rs:392-409 `rope_table`: theta = float32(pos) * frequency; cos, sin rounded to bf16.
inline void rope_cs(uint32_t pos, float freq, float& c, float& s) {
    const float theta = float(pos) * freq;
    c = round_bf16(std::cos(theta));
    s = round_bf16(std::sin(theta));
}
// kernels.metal:727-736 `norm_rope` without the norm: interleaved pairs, in place; cs [hd/2][2].
inline void rope_pairs(float* v, uint32_t hd, const float* cs) {
    for (uint32_t i = 0; i < hd / 2; i++) {
        const float c = cs[2 * i], s = cs[2 * i + 1], a0 = v[2 * i], a1 = v[2 * i + 1];
        v[2 * i] = c * a0 + s * a1;
        v[2 * i + 1] = c * a1 - s * a0;
    }
}

inline void inv_rms(const float* X, uint32_t n, uint32_t k, float eps, float* inv) {
    for (uint32_t t = 0; t < n; t++) {
        float ss = 0.0f;
        for (uint32_t i = 0; i < k; i++) ss += X[size_t(t) * k + i] * X[size_t(t) * k + i];
        inv[t] = 1.0f / std::sqrt(ss / float(k) + eps);
    }
}

}  // namespace orc
