// Shared host-side helpers: errors, device buffers, the structs mirrored on the GPU.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <cstdio>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace vlt {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define VLT_CUDA(call)                                                                                         \
    do {                                                                                                       \
        cudaError_t err__ = (call);                                                                            \
        if (err__ != cudaSuccess)                                                                              \
            throw ::vlt::Error(std::string(#call) + ": " + cudaGetErrorString(err__) + " (" __FILE__ ":" + std::to_string(__LINE__) + ")"); \
    } while (0)

// Kernels this library has launched (every launcher counts its own), for benchmarks to report.
// Atomic: engines on several threads and the engine-less entry points all count here.
inline std::atomic<uint64_t>& launch_counter() {
    static std::atomic<uint64_t> count{0};
    return count;
}

// Work that must happen once per CUDA device (cudaFuncSetAttribute applies to the current device only, and one
// process may hold engines on several devices): `once(f)` runs f the first time it is called with a given device
// current, under a lock, so that a second thread on the same device waits for the set-up instead of racing it.
class PerDevice {
  public:
    template <typename F>
    void once(F&& f) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
        std::lock_guard<std::mutex> lock(mu_);
        if ((done_ >> dev) & 1ull) return;
        f();
        done_ |= 1ull << dev;
    }

  private:
    std::mutex mu_;
    uint64_t done_ = 0;
};

// engine/src/engine/kernels.rs:14-29.
constexpr uint32_t FEED_ROW = 0xffff0000u;
constexpr uint32_t FEED_W = 16;
constexpr uint32_t NO_TOK = 0xffffffffu;
constexpr uint32_t VERIFY_T = 8;
constexpr uint32_t MAX_STOP = 8;
constexpr uint32_t NO_PARENT = 0xffu;

// engine/src/engine/kernels.rs:20-24 `chain_node`.
inline uint32_t chain_node(uint32_t row) {
    const uint32_t parent = row == 0 ? NO_PARENT : row - 1;
    return row | parent << 8 | ((2u << row) - 1u) << 16;
}

// engine/src/engine/kernels.rs:87-127: bit-compatible with the reference's #[repr(C)] structs.
struct SampleRow {
    uint32_t seed_lo, seed_hi;
    uint32_t pos;  // the drawn token's position, if tok is NO_TOK
    float temperature;
    float top_p;
    uint32_t tok;  // the step's token whose head row this is: the draw is at its position + 1
};
struct RunIn {
    uint32_t slot, first, count;
    uint32_t head0, nhead;
    uint32_t verify;
};
struct GenState {
    uint32_t remaining, done, nstop, pad;
    uint32_t stop[MAX_STOP];
};
inline GenState gen_open() { return GenState{0xffffffffu, 0, 0, 0, {0, 0, 0, 0, 0, 0, 0, 0}}; }
struct ReplayArgs {
    uint32_t stride, seed;
    float rate;
    uint32_t vocab;
};

// A buffer on the device, or on the host for a host-only (planning) engine. Written and read
// through explicit copies; step inputs use the pinned mirror for asynchronous uploads.
// `order`: the stream whose kernels use the buffer. With it set, write() and read() are copies on that stream
// (ordered against the kernels before and after them; a pageable source is staged before the call returns, so
// the caller may reuse it). Without it they are set-up copies that have landed when the call returns.
struct Buffer {
    void* dev = nullptr;
    size_t bytes = 0;
    bool host_only = false;
    cudaStream_t order = nullptr;

    Buffer() = default;
    Buffer(const Buffer&) = delete;
    Buffer& operator=(const Buffer&) = delete;
    Buffer(Buffer&& o) noexcept { *this = std::move(o); }
    Buffer& operator=(Buffer&& o) noexcept {
        release();
        dev = o.dev; bytes = o.bytes; host_only = o.host_only; order = o.order;
        o.dev = nullptr; o.bytes = 0;
        return *this;
    }
    ~Buffer() { release(); }

    void alloc(size_t n, bool host) {
        release();
        bytes = n;
        host_only = host;
        if (n == 0) return;
        if (host) {
            dev = std::calloc(1, n);
            if (!dev) throw Error("out of host memory");
        } else {
            VLT_CUDA(cudaMalloc(&dev, n));
            VLT_CUDA(cudaMemset(dev, 0, n));
        }
    }
    void release() {
        if (!dev) return;
        if (host_only) std::free(dev);
        else cudaFree(dev);
        dev = nullptr;
    }
    template <typename T> T* as() const { return static_cast<T*>(dev); }

    void write(size_t offset_bytes, const void* src, size_t n) const {
        if (n == 0) return;
        if (offset_bytes + n > bytes) throw Error("buffer write out of range");
        char* dst = static_cast<char*>(dev) + offset_bytes;
        if (host_only) {
            std::memcpy(dst, src, n);
        } else if (order) {
            VLT_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, order));
        } else {
            // A blocking copy from pageable memory may return once the bytes are staged, before the DMA lands, and
            // the engine's streams do not wait for the legacy stream: wait for it here.
            VLT_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice));
            VLT_CUDA(cudaStreamSynchronize(cudaStreamLegacy));
        }
    }
    void read(size_t offset_bytes, void* dst, size_t n) const {
        if (n == 0) return;
        if (offset_bytes + n > bytes) throw Error("buffer read out of range");
        const char* src = static_cast<const char*>(dev) + offset_bytes;
        if (host_only) {
            std::memcpy(dst, src, n);
        } else if (order) {
            VLT_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, order));
            VLT_CUDA(cudaStreamSynchronize(order));
        } else {
            VLT_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost));
        }
    }
    template <typename T> void write_vec(size_t index, const std::vector<T>& v) const { write(index * sizeof(T), v.data(), v.size() * sizeof(T)); }
    template <typename T> std::vector<T> read_vec(size_t index, size_t count) const {
        std::vector<T> v(count);
        read(index * sizeof(T), v.data(), count * sizeof(T));
        return v;
    }
};

#ifdef __CUDACC__
// A launch with programmatic stream serialization: the kernel may be scheduled while the one before it
// still runs; it must call pdl_start() before touching anything (every kernel launched this way does).
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VLT_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    launch_counter().fetch_add(1, std::memory_order_relaxed);
}
#endif

}  // namespace vlt
