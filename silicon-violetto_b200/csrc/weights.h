// The .vlt weight file, read into one device buffer, and the model's tensor table.
// Layout: tools/convert.py:117-133 (writer), engine/src/weights.rs:37-74 (reader).
#pragma once
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace vlt {

enum class DType : uint32_t { F32 = 0, Bf16 = 1, I8 = 2 };

struct Tensor {
    DType dtype;
    std::vector<uint32_t> shape;
    size_t offset, nbytes;  // offset into the weight buffer
};

struct Weights {
    Buffer buffer;
    std::map<std::string, Tensor> tensors;
    std::vector<uint8_t> host;  // small f32 tensors are also read on the host from here
    std::string path;

    // engine/src/weights.rs:38-74 `load`.
    void load(const std::string& p, bool host_only) {
        path = p;
        FILE* f = std::fopen(p.c_str(), "rb");
        if (!f) throw Error(p + ": cannot open");
        struct Closer { FILE* f; ~Closer() { std::fclose(f); } } closer{f};
        uint8_t head[32];
        if (std::fread(head, 1, 32, f) != 32) throw Error(p + ": short header");
        auto u32 = [](const uint8_t* b) { uint32_t v; std::memcpy(&v, b, 4); return v; };
        auto u64 = [](const uint8_t* b) { uint64_t v; std::memcpy(&v, b, 8); return v; };
        if (std::memcmp(head, "VIOLETTO", 8) != 0 || u32(head + 8) != 1) throw Error(p + ": not a version-1 violetto weight file");
        const uint32_t n = u32(head + 12);
        const uint64_t data_offset = u64(head + 16);
        std::vector<uint8_t> rec(size_t(128) * n);
        if (std::fread(rec.data(), 1, rec.size(), f) != rec.size()) throw Error(p + ": short tensor records");
        size_t end = 0;
        for (uint32_t i = 0; i < n; i++) {
            const uint8_t* r = rec.data() + size_t(128) * i;
            size_t len = 0;
            while (len < 64 && r[len]) len++;
            std::string name(reinterpret_cast<const char*>(r), len);
            const uint32_t d = u32(r + 64);
            if (d > 2) throw Error(name + ": unknown dtype " + std::to_string(d));
            Tensor t;
            t.dtype = DType(d);
            const uint32_t ndim = u32(r + 68);
            if (ndim > 4) throw Error(name + ": more than 4 dimensions");
            for (uint32_t j = 0; j < ndim; j++) t.shape.push_back(u32(r + 72 + 4 * j));
            t.offset = u64(r + 88);
            t.nbytes = u64(r + 96);
            end = std::max(end, t.offset + t.nbytes);
            tensors[name] = t;
        }
        // One buffer for everything (weights.rs:64-72), staged through pinned memory in slices.
        if (std::fseek(f, long(data_offset), SEEK_SET) != 0) throw Error(p + ": cannot seek to the data region");
        buffer.alloc(end, host_only);
        const size_t SLICE = size_t(64) << 20;
        std::vector<uint8_t> stage(std::min(end, SLICE));
        for (size_t at = 0; at < end; at += SLICE) {
            const size_t nb = std::min(SLICE, end - at);
            if (std::fread(stage.data(), 1, nb, f) != nb) throw Error(p + ": short data region");
            buffer.write(at, stage.data(), nb);
        }
        // Keep the small f32 tensors on the host too.
        for (auto& [name, t] : tensors)
            if (t.dtype == DType::F32 && t.nbytes <= (1u << 20)) {
                if (host.size() < t.offset + t.nbytes) host.resize(t.offset + t.nbytes);
                buffer.read(t.offset, host.data() + t.offset, t.nbytes);
            }
    }

    bool has(const std::string& name) const { return tensors.count(name) != 0; }
    const Tensor& tensor(const std::string& name) const {
        auto it = tensors.find(name);
        if (it == tensors.end()) throw Error("weight file has no tensor " + name);
        return it->second;
    }
    // engine/src/weights.rs:83-89 `get`.
    const Tensor& get(const std::string& name, DType dtype, const std::vector<uint32_t>& shape) const {
        const Tensor& t = tensor(name);
        if (t.dtype != dtype || t.shape != shape) {
            auto fmt = [](const std::vector<uint32_t>& s) { std::string o = "["; for (size_t i = 0; i < s.size(); i++) o += (i ? ", " : "") + std::to_string(s[i]); return o + "]"; };
            throw Error(name + ": expected dtype " + std::to_string(uint32_t(dtype)) + " " + fmt(shape) + ", found dtype " + std::to_string(uint32_t(t.dtype)) + " " + fmt(t.shape));
        }
        return t;
    }
    // engine/src/weights.rs:91-95 `f32s`.
    std::vector<float> f32s(const std::string& name) const {
        const Tensor& t = tensor(name);
        if (t.dtype != DType::F32) throw Error(name + ": expected f32");
        std::vector<float> v(t.nbytes / 4);
        if (t.offset + t.nbytes <= host.size()) std::memcpy(v.data(), host.data() + t.offset, t.nbytes);
        else buffer.read(t.offset, v.data(), t.nbytes);
        return v;
    }
};

// engine/src/model.rs:22-47 `Matrix`, `Int8`: [m][k] row-major at `w`; int8 has bf16 scales
// [m][k / group] at `scales`.
struct Matrix {
    const uint8_t* w = nullptr;
    const uint16_t* scales = nullptr;
    uint32_t m = 0, k = 0, group = 0;
    bool int8 = false;
    size_t bytes() const { return int8 ? size_t(m) * k + size_t(2) * m * (k / group) : size_t(2) * m * k; }
};

// engine/src/model.rs:81-103 `matrix`. The reference takes scale groups of 8..256; one scale per
// output row (group = k) is taken as well.
inline Matrix load_matrix(const Weights& w, const std::string& name, uint32_t m, uint32_t k) {
    const uint8_t* base = w.buffer.as<uint8_t>();
    Matrix out;
    out.m = m;
    out.k = k;
    if (w.tensor(name).dtype != DType::I8) {
        out.w = base + w.get(name, DType::Bf16, {m, k}).offset;
        return out;
    }
    out.w = base + w.get(name, DType::I8, {m, k}).offset;
    const std::string sn = name + ".scale";
    const Tensor& st = w.tensor(sn);
    const uint32_t groups = st.shape.size() > 1 ? st.shape[1] : 0;
    const uint32_t group = k / std::max(groups, 1u);
    // Groups of a power of two, or one scale per row whatever k is.
    if (group < 8 || (groups > 1 && (group & (group - 1))) || group * groups != k) throw Error(sn + ": " + std::to_string(groups) + " groups per row of " + std::to_string(k));
    out.scales = reinterpret_cast<const uint16_t*>(base + w.get(sn, DType::Bf16, {m, groups}).offset);
    out.group = group;
    out.int8 = true;
    return out;
}

struct ModelDesc {
    uint32_t n_layers = 0, d = 0, n_heads = 0, n_kv = 0, hd = 0, ffn = 0, vocab = 0, vocab_real = 0, page = 0;
    float eps = 0, attn_scale = 0;
    uint32_t qkv_w() const { return (n_heads + 2 * n_kv) * hd; }
    uint32_t group() const { return n_heads / n_kv; }
};

struct Layer {
    Matrix qkv, o, gate_up, down;
};

// What a layer of the reference's own architecture has beyond the four projections (engine/src/model.rs:49-67): device
// pointers into the weight buffer, and the scalars of tools/convert.py:104.
struct LimiteLayer {
    const float* attn_gate = nullptr;  // [n_heads][128]
    const float* ve_gate = nullptr;    // [n_kv][12]; layers with value embeddings only
    const float* xsa = nullptr;        // [n_heads]
    float qkv_scale = 1, o_scale = 1, resid_attn = 1, post_attn = 1, resid_mlp = 1, post_mlp = 1;
    bool global = false;
    uint32_t kv_index = 0;  // among the global or among the local layers
};

// engine/src/model.rs:69-155 `Model`: a plain decoder the file's `meta` describes, or -- a file of tools/convert.py, which
// has no `meta` -- the reference's own architecture (`limite`), whose shapes the reference fixes (model.rs:6-20) and
// which are read off the file here (heads stay 128 wide).
struct Model {
    Weights w;
    ModelDesc md;
    const uint16_t* embed = nullptr;  // bf16 [vocab][d], for the lookups
    Matrix head;                      // the embedding itself (tied) unless the file has a `head`
    std::vector<Layer> layers;
    std::vector<float> rope_freq;
    bool limite = false;
    std::vector<LimiteLayer> lim;
    const uint16_t* value_embed = nullptr;  // [vocab][n_kv * 128] bf16
    const float* mudd_dense1 = nullptr;     // [32][d]
    const float* mudd_mix = nullptr;        // [2][2][3][33]
    uint32_t n_local = 0, n_global = 0;

    void load(const std::string& path, bool host_only) {
        w.load(path, host_only);
        limite = !w.has("meta") && w.has("L00.scalars");
        if (limite) {
            const Tensor& et = w.tensor("embed");
            if (et.shape.size() != 2) throw Error(path + ": embed is not a matrix");
            md.vocab = et.shape[0]; md.d = et.shape[1]; md.hd = 128;
            if (md.d % 128) throw Error(path + ": hidden width is not a multiple of 128");
            md.n_heads = md.d / 128;
            md.n_kv = (w.tensor("L00.qkv").shape.at(0) / 128 - md.n_heads) / 2;
            md.ffn = w.tensor("L00.down").shape.at(1);
            md.n_layers = 0;
            while (w.has("L" + std::string(md.n_layers < 10 ? "0" : "") + std::to_string(md.n_layers) + ".qkv")) md.n_layers++;
            md.vocab_real = w.has("limite_vocab_real") ? uint32_t(w.f32s("limite_vocab_real").at(0)) : md.vocab == 151680 ? 151667u : md.vocab;
            md.eps = 0x1p-23f; md.page = 128; md.attn_scale = 0.1f;  // kernels.metal:13, kv.rs:6, model.rs:19
            if (md.n_kv == 0 || md.n_heads % md.n_kv || md.n_heads + md.n_kv > 32) throw Error(path + ": the qkv projection's rows do not fit the heads");
            if (md.n_layers < 4) throw Error(path + ": a model of this architecture has local and global layers (at least 4 layers)");
        } else {
        std::vector<float> m = w.f32s("meta");
        if (m.size() < 14 || m[0] != 1.0f || m[1] != 0.0f) throw Error(path + ": `meta` is not a version-1 plain-decoder descriptor");
        md.n_layers = uint32_t(m[2]); md.d = uint32_t(m[3]); md.n_heads = uint32_t(m[4]); md.n_kv = uint32_t(m[5]);
        md.hd = uint32_t(m[6]); md.ffn = uint32_t(m[7]); md.vocab = uint32_t(m[8]); md.vocab_real = uint32_t(m[9]);
        md.eps = m[10]; md.page = uint32_t(m[11]); md.attn_scale = m[13];
        if (md.hd != 64) throw Error(path + ": head_dim " + std::to_string(md.hd) + " (the attention kernels are built for 64)");
        if (md.page != 16) throw Error(path + ": page_size " + std::to_string(md.page) + " (the attention kernels are built for 16-token pages)");
        if (md.n_kv == 0 || md.n_heads % md.n_kv || md.group() > 4) throw Error(path + ": " + std::to_string(md.n_heads) + " query heads over " + std::to_string(md.n_kv) + " kv heads (at most 4 per kv head)");
        if (md.d % 256 || md.ffn % 256 || (md.n_heads * md.hd) % 256) throw Error(path + ": d_model, ffn and heads * head_dim must be multiples of 256");
        }
        embed = reinterpret_cast<const uint16_t*>(w.buffer.as<uint8_t>() + w.get("embed", DType::Bf16, {md.vocab, md.d}).offset);
        if (w.has("head")) head = load_matrix(w, "head", md.vocab, md.d);
        else { head.w = reinterpret_cast<const uint8_t*>(embed); head.m = md.vocab; head.k = md.d; }
        for (uint32_t i = 0; i < md.n_layers; i++) {
            char nm[40];
            auto name = [&](const char* k) { std::snprintf(nm, sizeof nm, "L%02u.%s", i, k); return std::string(nm); };
            Layer l;
            l.qkv = load_matrix(w, name("qkv"), md.qkv_w(), md.d);
            l.o = load_matrix(w, name("o"), md.d, md.n_heads * md.hd);
            l.gate_up = load_matrix(w, name("gate_up"), 2 * md.ffn, md.d);
            l.down = load_matrix(w, name("down"), md.d, md.ffn);
            layers.push_back(l);
            if (!limite) continue;
            const uint8_t* base = w.buffer.as<uint8_t>();
            auto f32 = [&](const char* k, std::vector<uint32_t> shape) { return reinterpret_cast<const float*>(base + w.get(name(k), DType::F32, shape).offset); };
            LimiteLayer x;  // model.rs:108-135
            x.global = i % 4 == 3;
            x.kv_index = x.global ? n_global++ : n_local++;
            x.attn_gate = f32("attn_gate", {md.n_heads, 128});
            if (i % 3 == 1) x.ve_gate = f32("ve_gate", {md.n_kv, 12});
            x.xsa = f32("xsa", {md.n_heads});
            f32("scalars", {8});
            const std::vector<float> sc = w.f32s(name("scalars"));
            x.qkv_scale = sc[0]; x.o_scale = sc[1]; x.resid_attn = sc[2]; x.post_attn = sc[3]; x.resid_mlp = sc[4]; x.post_mlp = sc[5];
            lim.push_back(x);
        }
        if (limite) {
            const uint8_t* base = w.buffer.as<uint8_t>();
            value_embed = reinterpret_cast<const uint16_t*>(base + w.get("value_embed", DType::Bf16, {md.vocab, md.n_kv * 128}).offset);
            mudd_dense1 = reinterpret_cast<const float*>(base + w.get("mudd.dense1", DType::F32, {32, md.d}).offset);
            mudd_mix = reinterpret_cast<const float*>(base + w.get("mudd.mix", DType::F32, {2, 2, 3, 33}).offset);
        }
        rope_freq = w.f32s("rope_freq");
        // (a head of 128 of the reference's architecture turns its first 64 dims: 32 pairs)
        if (rope_freq.size() != (limite ? 32 : md.hd / 2)) throw Error("rope_freq: expected head_dim / 2 entries (32 for the reference's own architecture)");
    }
};

}  // namespace vlt
