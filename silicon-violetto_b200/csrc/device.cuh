// Device-side helpers shared by the kernels: bf16 bits, Philox, the sampler's exp2, reductions.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace vlt {

// kernels.metal:17 `bf`.
__device__ __forceinline__ float bf16_to_f32(uint16_t u) { return __uint_as_float(uint32_t(u) << 16); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// kernels.metal:22-27 `to_bf`: round to nearest even. The hardware conversion gives the reference's integer formula's
// bits for every finite input (and a quiet NaN for NaN, where the formula would carry into the exponent); one
// instruction instead of five, two values at once in pack_bf16.
__device__ __forceinline__ uint16_t f32_to_bf16(float f) {
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}
__device__ __forceinline__ float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }
// Two floats to packed bf16 (lo in the low half), same rounding.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// kernels.metal:1462-1472 `philox`: Philox4x32-10.
__device__ __forceinline__ uint4 philox(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int i = 0; i < 10; i++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c;
}
// kernels.metal:1474-1477 `uniform01`.
__device__ __forceinline__ float uniform01(uint32_t seed_lo, uint32_t seed_hi, uint32_t pos, uint32_t round) {
    return __fmul_rn(float(philox(make_uint4(pos, round, 0, 0), seed_lo, seed_hi).x >> 8), 0x1p-24f);
}

// 2^x for the sampler, from IEEE operations only so that a draw is the same on every device
// and on the host: round x to the nearest integer n, a degree-6 polynomial in x - n on
// [-0.5, 0.5] by Horner with fused multiply-adds, n added to the exponent. 0 below 2^-125.
// (The reference calls Metal's exp2, kernels.metal:1536, whose last bits are the vendor's.)
__device__ __forceinline__ float soft_exp2(float x) {
    if (!(x > -125.5f)) return 0.0f;
    if (x > 126.0f) x = 126.0f;
    const float magic = 12582912.0f;
    const float t = __fadd_rn(x, magic);
    const int n = __float_as_int(t) - 0x4B400000;
    const float f = __fsub_rn(x, __fsub_rn(t, magic));
    float p = 0.00015403530393381608f;
    p = __fmaf_rn(p, f, 0.0013333558146428443f);
    p = __fmaf_rn(p, f, 0.009618129107628477f);
    p = __fmaf_rn(p, f, 0.05550410866482158f);
    p = __fmaf_rn(p, f, 0.2402265069591007f);
    p = __fmaf_rn(p, f, 0.6931471805599453f);
    p = __fmaf_rn(p, f, 1.0f);
    return __int_as_float(__float_as_int(p) + (n << 23));
}

// Two at once, on the packed fp32 instructions of sm_100 (add / mul / fma .f32x2: each half is the scalar IEEE operation, so
// each half's result is soft_exp2's, bit for bit). The samplers are bound by instruction issue, and this is most of it.
__device__ __forceinline__ float2 soft_exp2_x2(float2 x) {
    const bool zero0 = !(x.x > -125.5f), zero1 = !(x.y > -125.5f);
    x.x = fminf(x.x, 126.0f);
    x.y = fminf(x.y, 126.0f);
    const float2 magic = make_float2(12582912.0f, 12582912.0f), minus_magic = make_float2(-12582912.0f, -12582912.0f), minus_one = make_float2(-1.0f, -1.0f);
    const float2 t = __fadd2_rn(x, magic);
    const int n0 = __float_as_int(t.x) - 0x4B400000, n1 = __float_as_int(t.y) - 0x4B400000;
    const float2 f = __ffma2_rn(__fadd2_rn(t, minus_magic), minus_one, x);  // x - (t - magic): the product by -1 is exact, one rounding as in the subtraction
    float2 p = make_float2(0.00015403530393381608f, 0.00015403530393381608f);
    p = __ffma2_rn(p, f, make_float2(0.0013333558146428443f, 0.0013333558146428443f));
    p = __ffma2_rn(p, f, make_float2(0.009618129107628477f, 0.009618129107628477f));
    p = __ffma2_rn(p, f, make_float2(0.05550410866482158f, 0.05550410866482158f));
    p = __ffma2_rn(p, f, make_float2(0.2402265069591007f, 0.2402265069591007f));
    p = __ffma2_rn(p, f, make_float2(0.6931471805599453f, 0.6931471805599453f));
    p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
    return make_float2(zero0 ? 0.0f : __int_as_float(__float_as_int(p.x) + (n0 << 23)), zero1 ? 0.0f : __int_as_float(__float_as_int(p.y) + (n1 << 23)));
}
// e(x) = 2^((x - mx) c) for two logits, as the scalar soft_exp2(__fmul_rn(__fsub_rn(x, mx), c)) twice.
__device__ __forceinline__ float2 soft_exp2_scaled_x2(float x0, float x1, float mx, float c) {
    return soft_exp2_x2(__fmul2_rn(__fadd2_rn(make_float2(x0, x1), make_float2(-mx, -mx)), make_float2(c, c)));
}

constexpr float LOG2E = 1.44269504088896340736f;

// kernels.metal:64-72.
__device__ __forceinline__ uint32_t d_tree_node(uint32_t depth, uint32_t parent, uint32_t sees) { return depth | parent << 8 | sees << 16; }
// Programmatic dependent launch, first thing in a kernel started that way: let the kernel queued behind
// this one be scheduled early (it waits in turn), then wait for the kernel before this one to complete.
// From here on everything is ordered as if the kernels ran one after another; only launch latency overlaps.
// With -DVLT_STEP_PROBE (a developer's build, VLT_NVCC_FLAGS in build.py) every kernel that starts through pdl_start()
// leaves two time stamps of its first block, before and after the wait for its predecessor (tags 1 and 2), and
// the streamed matmul leaves more (3 / 4: the first / last block's end, 5: its main loop's start); vlt_engine_free prints them
// to stderr as "SP <ns> <tag> <blocks> <threads> <file>", which shows where a step's time goes between kernels.
#ifdef VLT_STEP_PROBE
}  // namespace vlt
#include <cstdio>
#include <vector>
namespace vlt {
static __device__ unsigned long long sp_buf[4 * 16384];
static __device__ unsigned int sp_n;
__device__ __forceinline__ unsigned long long sp_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Time stamps are taken where they belong and written later, several at once (the slot comes from an atomic whose
// round trip would otherwise sit in the measured path).
__device__ __forceinline__ void sp_write(const unsigned long long* t, const unsigned* tags, unsigned n) {
    const unsigned i0 = atomicAdd(&sp_n, n);
    for (unsigned j = 0; j < n; j++) {
        const unsigned i = i0 + j;
        if (i < 16384) { sp_buf[4 * i] = t[j]; sp_buf[4 * i + 1] = tags[j]; sp_buf[4 * i + 2] = gridDim.x * gridDim.y * gridDim.z; sp_buf[4 * i + 3] = blockDim.x; }
    }
}
__device__ __forceinline__ void pdl_start() {
    const bool me = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0;
    unsigned long long t[2];
    if (me) t[0] = sp_now();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (me) {
        t[1] = sp_now();
        const unsigned tags[2] = {1, 2};
        sp_write(t, tags, 2);
    }
}
inline std::vector<void (*)()>& sp_registry() { static std::vector<void (*)()> v; return v; }
static void sp_dump_tu() {
    static unsigned long long h[4 * 16384];
    unsigned n = 0;
    cudaMemcpyFromSymbol(&n, sp_n, 4);
    cudaMemcpyFromSymbol(h, sp_buf, sizeof(h));
    if (n > 16384) n = 16384;
    for (unsigned i = 0; i < n; i++) fprintf(stderr, "SP %llu %llu %llu %llu %s\n", h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3], __FILE__);
}
namespace { struct SpReg { SpReg() { sp_registry().push_back(&sp_dump_tu); } }; static SpReg sp_reg_instance; }
#define SP_TIME(var) var = sp_now()
#define SP_WRITE(t, tags, n) sp_write(t, tags, n)
#else
#define SP_TIME(var) do { } while (0)
#define SP_WRITE(t, tags, n) do { } while (0)
__device__ __forceinline__ void pdl_start() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif
__device__ __forceinline__ uint32_t d_chain_node(uint32_t row) { return d_tree_node(row, row == 0 ? 0xffu : row - 1, (2u << row) - 1u); }
__device__ __forceinline__ uint32_t d_dead_node(uint32_t row) { return d_tree_node(1, 0xffu, 1u | 1u << row); }
__device__ __forceinline__ uint32_t node_depth(uint32_t n) { return n & 0xffu; }
__device__ __forceinline__ uint32_t node_parent(uint32_t n) { return (n >> 8) & 0xffu; }
__device__ __forceinline__ uint32_t node_sees(uint32_t n) { return n >> 16; }

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

// kernels.metal:1418-1427 `better`, `simd_best`: (value, id) with ties to the lowest id.
__device__ __forceinline__ void better(float& bv, uint32_t& bi, float v, uint32_t i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}
__device__ __forceinline__ void warp_best(float& bv, uint32_t& bi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, v, i);
    }
}

// Where kv head g's row for cache position pos starts, in elements (kernels.metal:704-711,
// the paged layout): [layer][page][kv head][page_tok][head_dim].
struct KvArgs {
    uint32_t n_pages, max_pages, n_kv, page_shift, hd;
};
__device__ __forceinline__ size_t kv_row(const KvArgs& kv, uint32_t layer, const uint32_t* page_table, uint32_t slot, uint32_t g, uint32_t pos) {
    const uint32_t page = page_table[size_t(slot) * kv.max_pages + (pos >> kv.page_shift)];
    const uint32_t psize = 1u << kv.page_shift;
    return ((size_t(layer) * kv.n_pages + page) * kv.n_kv + g) * psize * kv.hd + size_t(pos & (psize - 1)) * kv.hd;
}

}  // namespace vlt
