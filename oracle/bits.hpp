// CPU oracle: scalar building blocks. TEST INFRASTRUCTURE ONLY: nothing that ships may
// include, link or call this directory; only the tests, the smoke check and the benchmark's
// CPU-baseline leg do.
//
// Every function restates a piece of the reference's shader math (Belluxx/silicon-violetto,
// engine/src/kernels.metal) or of its Rust host (engine/src/engine/*.rs); the file:line each
// one follows is given beside it.
//
// Parity status: UNPINNED. The reference ships no golden vectors for this path and neither
// Metal nor Rust runs here, so these routines are checked against each other, against the
// reference's importable Python tooling where one exists (tools/convert.py: the weight file
// layout and the int8 quantiser), and against cuRAND's Philox on the GPU.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace orc {

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// kernels.metal:17 `bf`: a bf16 widened to fp32.
inline float bf16_to_f32(uint16_t u) { return u2f(uint32_t(u) << 16); }
// kernels.metal:22-27 `to_bf`, plan.rs:176-179 `round_bf16`: round to nearest even, finite inputs.
inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// kernels.metal:1462-1472 `philox`: Philox4x32-10 with Random123's constants.
struct U4 { uint32_t x, y, z, w; };
inline U4 philox(U4 c, uint32_t k0, uint32_t k1) {
    for (int i = 0; i < 10; i++) {
        uint64_t p0 = uint64_t(0xD2511F53u) * c.x, p1 = uint64_t(0xCD9E8D57u) * c.z;
        uint32_t hi0 = uint32_t(p0 >> 32), lo0 = uint32_t(p0);
        uint32_t hi1 = uint32_t(p1 >> 32), lo1 = uint32_t(p1);
        c = U4{hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0};
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c;
}
// kernels.metal:1474-1477 `uniform01`: [0,1) on a 2^-24 grid, counter (pos, round, 0, 0).
inline float uniform01(uint32_t seed_lo, uint32_t seed_hi, uint32_t pos, uint32_t round) {
    return float(philox(U4{pos, round, 0, 0}, seed_lo, seed_hi).x >> 8) * 0x1p-24f;
}

// 2^x for the sampler. The reference calls Metal's exp2 (kernels.metal:1536,1553,1568), whose
// last bits are the GPU vendor's; a draw that must be reproduced bit for bit on another
// device needs one definition made of IEEE operations only. This is it: round x to the
// nearest integer n, a degree-6 polynomial in f = x - n on [-0.5, 0.5] evaluated by Horner
// with fused multiply-adds, then n added to the exponent field. Below 2^-125 the result is 0.
inline float soft_exp2(float x) {
    if (!(x > -125.5f)) return 0.0f;  // also -inf and NaN
    if (x > 126.0f) x = 126.0f;
    const float magic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to an integer
    float t = x + magic;
    int32_t n = int32_t(f2u(t)) - 0x4B400000;
    float f = x - (t - magic);
    float p = 0.00015403530393381608f;
    p = std::fmaf(p, f, 0.0013333558146428443f);
    p = std::fmaf(p, f, 0.009618129107628477f);
    p = std::fmaf(p, f, 0.05550410866482158f);
    p = std::fmaf(p, f, 0.2402265069591007f);
    p = std::fmaf(p, f, 0.6931471805599453f);
    p = std::fmaf(p, f, 1.0f);
    return u2f(uint32_t(int32_t(f2u(p)) + (n << 23)));
}

constexpr float LOG2E = 1.44269504088896340736f;

// kernels.metal:64-72 draft-tree nodes, engine/kernels.rs:20-24.
constexpr uint32_t FEED_ROW = 0xffff0000u;
constexpr uint32_t FEED_W = 16;
constexpr uint32_t NO_PARENT = 0xffu;
constexpr uint32_t NO_TOK = 0xffffffffu;
inline uint32_t tree_node(uint32_t depth, uint32_t parent, uint32_t sees) { return depth | parent << 8 | sees << 16; }
inline uint32_t chain_node(uint32_t row) { return tree_node(row, row == 0 ? NO_PARENT : row - 1, (2u << row) - 1u); }
inline uint32_t dead_node(uint32_t row) { return tree_node(1, NO_PARENT, 1u | 1u << row); }
inline uint32_t node_depth(uint32_t n) { return n & 0xffu; }
inline uint32_t node_parent(uint32_t n) { return (n >> 8) & 0xffu; }
inline uint32_t node_sees(uint32_t n) { return n >> 16; }

// engine/kernels.rs:87-127, mirrored by kernels.metal:1454-1460,1590-1602.
struct SampleRow {
    uint32_t seed_lo, seed_hi;
    uint32_t pos;
    float temperature;
    float top_p;
    uint32_t tok;
};
struct RunIn {
    uint32_t slot, first, count;
    uint32_t head0, nhead;
    uint32_t verify;
};
constexpr uint32_t MAX_STOP = 8;
struct GenState {
    uint32_t remaining, done, nstop, pad;
    uint32_t stop[MAX_STOP];
};

}  // namespace orc
