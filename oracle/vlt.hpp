// CPU oracle (test infrastructure only, parity unpinned: see bits.hpp): the .vlt weight file
// and the int8 quantiser. Pinned against the reference's own tools/convert.py (`write`,
// `read`, `quantize`), which imports in this environment: tests/golden holds files and
// vectors it produced.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "bits.hpp"

namespace orc {

enum DType : uint32_t { F32 = 0, BF16 = 1, I8 = 2 };

struct Tensor {
    std::string name;
    DType dtype;
    std::vector<uint32_t> shape;
    uint64_t offset, nbytes;  // offset from the start of the data region
};

// engine/src/weights.rs:37-74 `Weights::load`; layout documented at tools/convert.py:117-133.
struct VltFile {
    std::vector<Tensor> tensors;           // in file order
    std::map<std::string, size_t> by_name;
    std::vector<uint8_t> data;             // the data region up to the last tensor's end

    static VltFile load(const std::string& path) {
        FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) throw std::runtime_error(path + ": cannot open");
        uint8_t head[32];
        if (std::fread(head, 1, 32, f) != 32) { std::fclose(f); throw std::runtime_error(path + ": short header"); }
        auto u32 = [](const uint8_t* b) { uint32_t v; std::memcpy(&v, b, 4); return v; };
        auto u64 = [](const uint8_t* b) { uint64_t v; std::memcpy(&v, b, 8); return v; };
        if (std::memcmp(head, "VIOLETTO", 8) != 0 || u32(head + 8) != 1) {
            std::fclose(f);
            throw std::runtime_error(path + ": not a version-1 violetto weight file");
        }
        const uint32_t n = u32(head + 12);
        const uint64_t data_offset = u64(head + 16);
        std::vector<uint8_t> rec(size_t(128) * n);
        if (std::fread(rec.data(), 1, rec.size(), f) != rec.size()) { std::fclose(f); throw std::runtime_error(path + ": short records"); }
        VltFile out;
        uint64_t end = 0;
        for (uint32_t i = 0; i < n; i++) {
            const uint8_t* r = rec.data() + size_t(128) * i;
            size_t len = 0;
            while (len < 64 && r[len]) len++;
            Tensor t;
            t.name.assign(reinterpret_cast<const char*>(r), len);
            const uint32_t d = u32(r + 64);
            if (d > 2) { std::fclose(f); throw std::runtime_error(t.name + ": unknown dtype"); }
            t.dtype = DType(d);
            const uint32_t ndim = u32(r + 68);
            for (uint32_t j = 0; j < ndim && j < 4; j++) t.shape.push_back(u32(r + 72 + 4 * j));
            t.offset = u64(r + 88);
            t.nbytes = u64(r + 96);
            end = std::max(end, t.offset + t.nbytes);
            out.by_name[t.name] = out.tensors.size();
            out.tensors.push_back(t);
        }
        out.data.resize(end);
        std::fseek(f, long(data_offset), SEEK_SET);
        if (std::fread(out.data.data(), 1, end, f) != end) { std::fclose(f); throw std::runtime_error(path + ": short data region"); }
        std::fclose(f);
        return out;
    }

    bool has(const std::string& name) const { return by_name.count(name) != 0; }
    const Tensor& tensor(const std::string& name) const {
        auto it = by_name.find(name);
        if (it == by_name.end()) throw std::runtime_error("weight file has no tensor " + name);
        return tensors[it->second];
    }
    // engine/src/weights.rs:83-89 `get`: dtype and shape must match.
    const Tensor& get(const std::string& name, DType dtype, const std::vector<uint32_t>& shape) const {
        const Tensor& t = tensor(name);
        if (t.dtype != dtype || t.shape != shape) throw std::runtime_error(name + ": unexpected dtype or shape");
        return t;
    }
    const uint8_t* ptr(const Tensor& t) const { return data.data() + t.offset; }
    std::vector<float> f32s(const std::string& name) const {
        const Tensor& t = tensor(name);
        if (t.dtype != F32) throw std::runtime_error(name + ": not f32");
        std::vector<float> v(t.nbytes / 4);
        std::memcpy(v.data(), ptr(t), t.nbytes);
        return v;
    }
};

// tools/convert.py:117-152 `write`: tensors 256-byte aligned in a 16 KiB aligned data region.
struct VltWriter {
    struct Item { std::string name; DType dtype; std::vector<uint32_t> shape; std::vector<uint8_t> raw; };
    std::vector<Item> items;
    void add(const std::string& name, DType dtype, const std::vector<uint32_t>& shape, const void* p, size_t nbytes) {
        Item it{name, dtype, shape, {}};
        it.raw.assign(static_cast<const uint8_t*>(p), static_cast<const uint8_t*>(p) + nbytes);
        items.push_back(std::move(it));
    }
    void write(const std::string& path) const {
        const uint64_t TA = 256, DA = 16384;
        std::vector<uint8_t> rec(items.size() * 128, 0);
        std::vector<uint64_t> offs;
        uint64_t off = 0;
        for (size_t i = 0; i < items.size(); i++) {
            const Item& it = items[i];
            off = (off + TA - 1) / TA * TA;
            uint8_t* r = rec.data() + 128 * i;
            std::memcpy(r, it.name.data(), std::min<size_t>(it.name.size(), 63));
            uint32_t d = it.dtype, nd = uint32_t(it.shape.size());
            std::memcpy(r + 64, &d, 4);
            std::memcpy(r + 68, &nd, 4);
            for (uint32_t j = 0; j < nd; j++) std::memcpy(r + 72 + 4 * j, &it.shape[j], 4);
            uint64_t nb = it.raw.size();
            std::memcpy(r + 88, &off, 8);
            std::memcpy(r + 96, &nb, 8);
            offs.push_back(off);
            off += nb;
        }
        const uint64_t header_len = 32 + rec.size();
        const uint64_t data_offset = (header_len + DA - 1) / DA * DA;
        const uint64_t total = data_offset + (off + DA - 1) / DA * DA;
        std::vector<uint8_t> file(total, 0);
        std::memcpy(file.data(), "VIOLETTO", 8);
        uint32_t ver = 1, n = uint32_t(items.size());
        std::memcpy(file.data() + 8, &ver, 4);
        std::memcpy(file.data() + 12, &n, 4);
        std::memcpy(file.data() + 16, &data_offset, 8);
        std::memcpy(file.data() + 32, rec.data(), rec.size());
        for (size_t i = 0; i < items.size(); i++)
            std::memcpy(file.data() + data_offset + offs[i], items[i].raw.data(), items[i].raw.size());
        FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) throw std::runtime_error(path + ": cannot create");
        std::fwrite(file.data(), 1, file.size(), f);
        std::fclose(f);
    }
};

// tools/convert.py:41-50 `quantize`: s = bf16(absmax / 127) per group of `group` consecutive
// k; q = round_half_even(w / float(s)) clamped to +-127, 0 where s is 0.
inline void quantize(const float* w, uint32_t m, uint32_t k, uint32_t group, int8_t* q, uint16_t* s) {
    const uint32_t ng = k / group;
    for (uint32_t r = 0; r < m; r++) {
        for (uint32_t g = 0; g < ng; g++) {
            const float* x = w + uint64_t(r) * k + g * group;
            float amax = 0.0f;
            for (uint32_t i = 0; i < group; i++) amax = std::max(amax, std::fabs(x[i]));
            const uint16_t sb = f32_to_bf16(amax / 127.0f);
            const float sf = bf16_to_f32(sb);
            s[uint64_t(r) * ng + g] = sb;
            for (uint32_t i = 0; i < group; i++) {
                float v = sf > 0.0f ? std::nearbyintf(x[i] / sf) : 0.0f;
                v = std::min(127.0f, std::max(-127.0f, v));
                q[uint64_t(r) * k + g * group + i] = int8_t(v);
            }
        }
    }
}

}  // namespace orc
