// TEST INFRASTRUCTURE (CPU oracle, parity unpinned: the reference's target model has no Python definition in its tree --
// tools/common.py loads it from a checkpoint repository with trust_remote_code -- and its Metal kernels do not run here).
//
// The reference's own architecture ("Limite"), which its engine hard-codes (engine/src/model.rs:6-20): what a weight file
// of tools/convert.py:64-114 holds beyond the four projections of a layer, and the state its local layers keep. The
// forward pass over it is limite_forward.hpp. The reference fixes hidden 1280, 10 query / 2 kv heads of 128, FFN 3328,
// 48 layers, 151 680 ids; here the hidden width, the kv heads, the FFN, the layer count and the vocabulary come from
// the file (heads stay 128 wide), so that small models of the same graph can be tested:
//   - layer i is global (paged cache, no RoPE) if i % 4 == 3, else local (a ring of window + max_chunk positions per
//     slot, RoPE on the first 64 dims)                                     model.rs:113, encode.rs:227, kv.rs:26-33
//   - layers with i % 3 == 1 add gated value embeddings to v               model.rs:126, kernels.metal:738-747
//   - every layer: q/k RMS-norm per head, an attention gate per head, XSA, matrix scales and residual lambdas
//                                                                          kernels.metal:725-801,1314-1362, model.rs:127-132
//   - layers 24 and 47 mix the embedding, the output of layer 11 (22) and the current stream into the attention input
//     and the residual base (MUDD)                                         encode.rs:107-160, kernels.metal:1364-1407
//   - logits through 23 sigmoid((x + 5) / 7.5), padding ids masked         kernels.metal:196-199
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "linear.hpp"

namespace orc {

struct LimiteLayer {
    const float* attn_gate = nullptr;  // [n_heads][128]
    const float* ve_gate = nullptr;    // [n_kv][12], layers with value embeddings
    const float* xsa = nullptr;        // [n_heads]
    float qkv_scale = 1, o_scale = 1, resid_attn = 1, post_attn = 1, resid_mlp = 1, post_mlp = 1;
    bool global = false;
    uint32_t kv_index = 0;  // among the global or among the local layers
};

struct Limite {
    static constexpr uint32_t D = 128, WINDOW = 1024, PAGE = 128;
    static constexpr float XSA_EPS = 1e-4f;
    std::vector<LimiteLayer> layers;
    const uint16_t* value_embed = nullptr;  // [vocab][n_kv * 128] bf16
    const float* mudd_dense1 = nullptr;     // [32][hidden]
    const float* mudd_mix = nullptr;        // [2 sites][attention input, residual base][3 taps][32 weights + bias]
    uint32_t n_local = 0, n_global = 0, ring = 0, max_seqs = 0;
    std::vector<uint16_t> k_local, v_local;  // [local layer][slot][kv head][ring][128]

    static bool is_limite(const VltFile& f) { return !f.has("meta") && f.has("L00.scalars"); }
    static int mudd_site(uint32_t li) { return li == 24 ? 0 : li == 47 ? 1 : -1; }

    void init_state(uint32_t seqs, uint32_t max_chunk, uint32_t n_kv) {
        max_seqs = seqs;
        ring = WINDOW + max_chunk;  // kv.rs:26-28
        k_local.assign(size_t(n_local) * seqs * n_kv * ring * D, 0);
        v_local.assign(k_local.size(), 0);
    }
};

}  // namespace orc
