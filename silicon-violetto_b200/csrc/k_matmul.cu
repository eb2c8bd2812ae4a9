// Matmuls for steps of at most 8 tokens: weights streamed once from HBM into registers and
// multiplied on the tensor cores (the reference's "stream" GEMM, kernels.metal:516-690, and its
// GEMV, :211-317), plus a scalar kernel for any shape (cross-check, odd scale groups).
//
// Y[t][row] = epilogue(W[row] . bf16(X[t])), W [m][k] row-major bf16 or int8 with bf16 scales
// per group of consecutive k, X fp32 [n][k]. 1/rms(X[t]) is accumulated in the same pass
// (kernels.metal:239-251,286), so a folded RMSNorm costs no extra kernel.
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.h"

namespace vlt {

// kernels.metal:184-209 `epilogue`, `epilogue_swiglu`. A plain decoder's scales and residual lambdas are 1 and its head has
// no cap; the reference's own architecture sets them and takes EPI_HEAD_CAP.
__device__ __forceinline__ void store_out(const MatArgs& a, uint32_t t, uint32_t row, float acc, float inv) {
    const size_t o = size_t(t) * a.m + row;
    float y;
    switch (a.epi) {
    case EPI_NORM: y = acc * inv * a.scale; break;
    case EPI_RESID: y = a.ra * a.base[o] + a.rb * (a.scale * acc); break;
    case EPI_HEAD: y = row < a.vocab_real ? acc * inv : -INFINITY; break;
    case EPI_HEAD_CAP: y = row < a.vocab_real ? 23.0f * (1.0f / (1.0f + expf(-(acc + 5.0f) / 7.5f))) : -INFINITY; break;
    default: y = acc; break;
    }
    a.Y[o] = y;
    if (a.Yb) a.Yb[o] = f32_to_bf16(y);
}
__device__ __forceinline__ void store_swiglu(const MatArgs& a, uint32_t t, uint32_t row, float g, float u, float inv) {
    g *= inv;
    u *= inv;
    const float y = g * (1.0f / (1.0f + expf(-g))) * u;
    const size_t o = size_t(t) * (a.m / 2) + row / 2;
    a.Y[o] = y;
    if (a.Yb) a.Yb[o] = f32_to_bf16(y);
}

// ------------------------------------------------------------------ scalar
// One warp per pair of rows (a gate/up pair under SWIGLU), all tokens in blocks of 8.
__global__ void __launch_bounds__(256) matmul_rows_kernel(MatArgs a) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t row0 = (blockIdx.x * 8 + warp) * 2;
    if (row0 >= a.m) return;
    const uint32_t group = a.int8 ? a.group : a.k, ng = a.k / group;
    for (uint32_t t0 = 0; t0 < a.n; t0 += 8) {
        float acc[2][8], ss[8];
#pragma unroll
        for (int b = 0; b < 8; b++) { acc[0][b] = acc[1][b] = 0.0f; ss[b] = 0.0f; }
        for (uint32_t k0 = lane * 8; k0 < a.k; k0 += 256) {
            float w[2][8];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const size_t e = size_t(row0 + r) * a.k + k0;
                float sc = 1.0f;
                if (a.int8) {
                    const uint2 q = *reinterpret_cast<const uint2*>(a.W + e);
                    const int8_t* qb = reinterpret_cast<const int8_t*>(&q);
#pragma unroll
                    for (int i = 0; i < 8; i++) w[r][i] = float(qb[i]);
                    sc = bf16_to_f32(a.scales[size_t(row0 + r) * ng + k0 / group]);
                } else {
                    const uint4 q = *reinterpret_cast<const uint4*>(a.W + 2 * e);
                    w[r][0] = bf16lo(q.x); w[r][1] = bf16hi(q.x); w[r][2] = bf16lo(q.y); w[r][3] = bf16hi(q.y);
                    w[r][4] = bf16lo(q.z); w[r][5] = bf16hi(q.z); w[r][6] = bf16lo(q.w); w[r][7] = bf16hi(q.w);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) w[r][i] *= sc;  // exact: an int8 times a bf16 fits in fp32
            }
#pragma unroll
            for (int b = 0; b < 8; b++) {
                if (t0 + b >= a.n) break;
                const float4* xp = reinterpret_cast<const float4*>(a.X + size_t(t0 + b) * a.k + k0);
                const float4 xa = xp[0], xb = xp[1];
                const float x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    ss[b] += x[i] * x[i];
                    const float xr = round_bf16(x[i]);
                    acc[0][b] += w[0][i] * xr;
                    acc[1][b] += w[1][i] * xr;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 8; b++) {
            if (t0 + b >= a.n) break;
            const float s0 = warp_sum(acc[0][b]), s1 = warp_sum(acc[1][b]), sq = warp_sum(ss[b]);
            if (lane != 0) continue;
            const uint32_t t = t0 + b;
            const float inv = a.inv_in ? a.inv_in[t] : rsqrtf(sq / float(a.k) + a.eps);
            if (a.inv_out && row0 == 0) a.inv_out[t] = inv;
            if (a.epi == EPI_SWIGLU) store_swiglu(a, t, row0, s0, s1, inv);
            else { store_out(a, t, row0, s0, inv); store_out(a, t, row0 + 1, s1, inv); }
        }
    }
}

void launch_matmul_rows(const MatArgs& a, cudaStream_t s) {
    { matmul_rows_kernel<<<(a.m / 2 + 7) / 8, 256, 0, s>>>(a); launch_counter()++; }
}

// ---------------------------------------------------------- streamed, n <= 8
// Four int8 (one word) to two bf16 pairs, exactly: byte ^ 0x80 placed in the mantissa of 2^23
// gives 2^23 + 128 + q; subtracting that offset leaves q as an fp32 integer whose upper half is
// its bf16.
__device__ __forceinline__ void cvt_i8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
    lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
    hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four int8 (one word) to two fp16 pairs, exactly, in five instructions: byte ^ 0x80 under the exponent byte 0x64 is
// the half 1024 + 128 + q, and a packed subtraction of 1152 leaves q.
__device__ __forceinline__ void cvt_i8x4_f16(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t a = __byte_perm(u, 0x64646464u, 0x5140), b = __byte_perm(u, 0x64646464u, 0x5342);
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(0x64806480u));
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(0x64806480u));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- shared-memory pipeline pieces (bounded waits: a copy that never lands sets the error word instead of hanging)
__device__ __forceinline__ uint32_t st_smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void st_mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void st_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool st_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The whole warp waits (call it converged): one lane polls, so that a waiting block leaves the issue slots to the block
// it shares the SM with, then every lane observes the completed phase itself. False if the limit ran out.
__device__ __forceinline__ bool st_mbar_wait(uint32_t bar, uint32_t parity) {
    bool ok = true;
    if (threadIdx.x % 32 == 0) {
        ok = false;
        for (uint32_t i = 0; i < (1u << 22) && !ok; i++) ok = st_mbar_try(bar, parity);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok && st_mbar_try(bar, parity);
}
__device__ __forceinline__ void st_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// One resident block of 16 warps per `slot` walks over tiles of 16 weight rows (tile = block, + grid, ...). A row
// tile is cut along k into slices of at most 2 KiB per row; a (row tile, slice) is one item of the block's pipeline:
// its 16 row pieces come by bulk copy into a stage of shared memory (rows 64 bytes apart from a multiple of 128, so
// that the eight rows a quarter-warp reads fall in different banks), `n_stages` items ahead of the multiplication,
// and the first of them before the kernel waits for its predecessor (weights do not depend on it): HBM latency is
// paid once per launch, and the warps' meeting after each row tile does not stop the stream.
// Within a slice the 64-byte k tiles go to the warps in turn. A lane reads 16 bytes of row g and of row g + 8
// (g = lane / 4); since the contraction index may be permuted freely, lane t's consecutive k are used as k-slots
// (2t, 2t+1, 2t+8, 2t+9) of successive mma steps for A and B alike. The warps' sums meet in shared memory in warp order.
// The activations are staged once per block as bf16 ([n tokens][k], rows padded by 16 bytes against bank conflicts),
// their sums of squares for the folded RMSNorm taken in the same pass.
// int8 weights are multiplied as fp16 (the conversion above costs half the instructions of the one to bf16, and
// instruction issue is what bounds this kernel once the weights stream): the staged activations, already rounded to
// bf16, are then rewritten as fp16 times a power of two per token that puts the token's largest magnitude at 2^14,
// so nothing overflows and every bf16 value down to 2^-31 of the largest is still exact; the token's sums are
// multiplied back by the inverse power, which commutes with fp32 rounding: the products and sums are those of the
// bf16 form.
constexpr uint32_t STREAM_SLICE = 2048;                      // bytes of a weight row per item
constexpr uint32_t STREAM_ROW = STREAM_SLICE + 64;           // a stage's row stride
constexpr uint32_t STREAM_STAGE = 16 * STREAM_ROW;
constexpr uint32_t STREAM_MAX_STAGES = 6;
constexpr uint32_t STREAM_SCALE_TILES = 32;
constexpr uint32_t STREAM_AHEAD = 4;  // items asked of L2 ahead of the stages
constexpr size_t STREAM_SMEM_MAX = 216 * 1024;  // dynamic shared memory of a block (the kernel's static arrays take a few KiB more of the 227)

template <bool INT8>
__global__ void __launch_bounds__(512, 2) matmul_stream_kernel(MatArgs a, uint32_t n_stages) {
    constexpr int NW = 16;
    constexpr int E = INT8 ? 16 : 8;  // weights per 16-byte load
    constexpr int KS = E / 4;         // mma steps per 64-byte tile
    constexpr uint32_t WB = INT8 ? 1 : 2;
    extern __shared__ __align__(128) uint8_t stream_smem[];
    __shared__ uint64_t bars[STREAM_MAX_STAGES + 1];  // the stages', then the staged activations' (bf16 input only)
    __shared__ float ss_part[NW][8];
    __shared__ float mx_part[NW][8];
    __shared__ float x_down[8], x_up[8];  // int8: the power of two a token's activations are staged with, and its inverse
    __shared__ float row_scale[STREAM_SCALE_TILES * 16];  // one scale per row: the block's first row tiles' (the rest are read when needed)
    __shared__ float inv_s[8];
    __shared__ uint32_t rescale_s;
    __shared__ float2 q_cs[8][32];  // EPI_QKV: a token's (cos, sin) per pair of dims (head_dim <= 64)
    __shared__ size_t q_kvrow[8];   // EPI_QKV: a token's row in the cache for kv head 0 (~0: not written)
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane >> 2, t = lane & 3;
    const uint32_t xrs = a.k * 2 + 16;                                         // bytes per staged activation row
    uint8_t* stages = stream_smem;                                             // [n_stages][16][STREAM_ROW]
    float* red = reinterpret_cast<float*>(stream_smem + n_stages * STREAM_STAGE);  // [2][NW][16 rows][8 tokens]
    uint8_t* xs = reinterpret_cast<uint8_t*>(red + 2 * NW * 128);              // [n][xrs]
    const uint32_t row_bytes = a.k * WB, n_tiles = row_bytes / 64, n_row_tiles = a.m / 16;
    const uint32_t slices = (n_tiles + 31) / 32;
    const uint32_t my_row_tiles = (n_row_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const uint32_t n_items = my_row_tiles * slices;
    const bool grouped = INT8 && a.group < a.k;
    const uint32_t ng = INT8 ? a.k / a.group : 1;

    if (tid == 0) {
        for (uint32_t i = 0; i < n_stages; i++) st_mbar_init(st_smem_u32(&bars[i]), 1);
        st_mbar_init(st_smem_u32(&bars[STREAM_MAX_STAGES]), 1);
        rescale_s = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // One warp requests an item: lane 0 announces the bytes, lanes 0..15 copy a row piece each.
    auto request = [&](uint32_t item) {
        const uint32_t rt = blockIdx.x + (item / slices) * gridDim.x, sl = item % slices, st = item % n_stages;
        const uint32_t bytes = (min(n_tiles - sl * 32, 32u)) * 64, bar = st_smem_u32(&bars[st]);
        if (lane == 0) st_mbar_expect_tx(bar, bytes * 16);
        __syncwarp();
        if (lane < 16)
            st_bulk_load(st_smem_u32(stages + size_t(st) * STREAM_STAGE + lane * STREAM_ROW), a.W + size_t(rt * 16 + lane) * row_bytes + size_t(sl) * STREAM_SLICE, bytes, bar);
    };
    [[maybe_unused]] unsigned long long sp_t[4] = {0, 0, 0, 0};
    if (tid == 0) SP_TIME(sp_t[0]);
    // Another warp asks L2 for an item some items before it is asked for into a stage: a block that is resident early
    // (while the kernel before still runs) then has HBM work on more than its stages hold.
    auto prefetch = [&](uint32_t item) {
        const uint32_t rt = blockIdx.x + (item / slices) * gridDim.x, sl = item % slices;
        const uint32_t bytes = (min(n_tiles - sl * 32, 32u)) * 64;
        if (lane < 16) {
            const uint8_t* src = a.W + size_t(rt * 16 + lane) * row_bytes + size_t(sl) * STREAM_SLICE;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
        }
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // (The requesting warps are not among the four that add up and store a row tile: asking takes a while.)
    if (warp == NW - 1)
        for (uint32_t i = 0; i < min(n_stages, n_items); i++) request(i);
    if (warp == NW - 2)
        for (uint32_t i = n_stages; i < min(n_stages + STREAM_AHEAD, n_items); i++) prefetch(i);
    // The rows' scales are read once each, so every row tile would wait for HBM in its turn: all of them now.
    if (INT8 && !grouped)
        for (uint32_t i = tid; i < min(my_row_tiles, STREAM_SCALE_TILES) * 16; i += 512)
            row_scale[i] = bf16_to_f32(a.scales[(blockIdx.x + (i / 16) * gridDim.x) * 16 + i % 16]);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) SP_TIME(sp_t[1]);

    // ---- the activations into shared memory, in one pass.
    // int8 weights multiply as fp16: the values, rounded to bf16 first, are written as fp16 as they are while every
    // token's largest magnitude lies in [2^-6, 2^15) (nothing overflows, and what fp16 cannot hold exactly is below
    // 2^-19 of the largest); otherwise a second pass below rewrites all of them times a power of two per token.
    const uint32_t n4 = a.k / 4, total = a.n * n4;
    auto put = [&](uint32_t tk, uint32_t c, uint32_t p0, uint32_t p1, float down) {  // four bf16 values (two packed pairs) of token tk
        uint2* dst = reinterpret_cast<uint2*>(xs + size_t(tk) * xrs) + c;
        if (INT8) {
            const __half2 h0 = __floats2half2_rn(bf16lo(p0) * down, bf16hi(p0) * down), h1 = __floats2half2_rn(bf16lo(p1) * down, bf16hi(p1) * down);
            *dst = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        } else {
            *dst = make_uint2(p0, p1);
        }
    };
    auto magnitude = [](uint32_t p0, uint32_t p1) { return fmaxf(fmaxf(fabsf(bf16lo(p0)), fabsf(bf16hi(p0))), fmaxf(fabsf(bf16lo(p1)), fabsf(bf16hi(p1)))); };
    // The qkv epilogue's per-token values (position's rotation, cache row) are fetched by warps 8..15 meanwhile: their
    // chain of dependent loads (token -> position -> table) would otherwise follow the multiplication.
    if (a.epi == EPI_QKV && tid >= 256) {
        const uint32_t tk = (tid - 256) / 32, pair = (tid - 256) % 32, hd = a.q.kv.hd;
        if (tk < a.n) {
            const uint32_t tt = a.t0 + tk, pos = a.q.meta[2 * tt + 1];
            if (pair < hd / 2) q_cs[tk][pair] = reinterpret_cast<const float2*>(a.q.rope)[size_t(pos) * (hd / 2) + pair];
            if (pair == 0) {
                const uint32_t slot = a.q.meta[2 * tt], run_row = a.q.tin[2 * tt + 1];
                const uint32_t cpos = a.q.cpos ? a.q.cpos[tt] : a.q.meta[2 * (tt - run_row) + 1] + run_row;
                q_kvrow[tk] = cpos == NO_TOK ? ~size_t(0) : kv_row(a.q.kv, a.q.layer, a.q.page_table, slot, 0, cpos);
            }
        }
    }
    float ssb[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    float mxb[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (a.Xb) {
        // A bf16 copy left by the kernel before (this matrix folds no RMSNorm: no sum of squares): a bulk copy per token.
        const uint32_t xbar = st_smem_u32(&bars[STREAM_MAX_STAGES]);
        if (warp == 0) {
            if (lane == 0) st_mbar_expect_tx(xbar, a.n * a.k * 2);
            __syncwarp();
            if (lane < a.n) st_bulk_load(st_smem_u32(xs + size_t(lane) * xrs), a.Xb + size_t(lane) * a.k, a.k * 2, xbar);
        }
        if (INT8) {  // bf16 -> fp16 in place
            if (!st_mbar_wait(xbar, 0) && lane == 0 && a.err_flag) atomicExch(a.err_flag, 2u);
            // (the token loop is unrolled, so a token's accumulators are registers and no index is divided)
            for (uint32_t c = tid; c < n4; c += 512) {
#pragma unroll
                for (int tk = 0; tk < 8; tk++) {
                    if (uint32_t(tk) >= a.n) break;
                    const uint2 v = reinterpret_cast<const uint2*>(xs + size_t(tk) * xrs)[c];
                    mxb[tk] = fmaxf(mxb[tk], magnitude(v.x, v.y));
                    put(tk, c, v.x, v.y, 1.0f);
                }
            }
        }
    } else {
        // fp32 [n][k]: a float4 of every token per thread and step, the tokens' loads in flight together; a sum of
        // squares per token (the token loop is unrolled: a token's accumulators are registers).
        const float4* src = reinterpret_cast<const float4*>(a.X);
        for (uint32_t c = tid; c < n4; c += 512) {
            float4 v[8];
#pragma unroll
            for (int tk = 0; tk < 8; tk++) v[tk] = uint32_t(tk) < a.n ? src[size_t(tk) * n4 + c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int tk = 0; tk < 8; tk++) {
                if (uint32_t(tk) >= a.n) break;
                ssb[tk] += v[tk].x * v[tk].x + v[tk].y * v[tk].y + v[tk].z * v[tk].z + v[tk].w * v[tk].w;
                const uint32_t p0 = pack_bf16(v[tk].x, v[tk].y), p1 = pack_bf16(v[tk].z, v[tk].w);
                if (INT8) mxb[tk] = fmaxf(mxb[tk], magnitude(p0, p1));
                put(tk, c, p0, p1, 1.0f);
            }
        }
    }
#pragma unroll
    for (int b = 0; b < 8; b++) {
        float ss = ssb[b], mx = mxb[b];
        if (uint32_t(b) < a.n) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                if (!a.Xb) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (INT8) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
        }
        if (lane == 0) { ss_part[warp][b] = ss; mx_part[warp][b] = mx; }
    }
    __syncthreads();
    if (tid < 8) {
        float block_ss = 0.0f, mx = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++) { block_ss += ss_part[w][tid]; mx = fmaxf(mx, mx_part[w][tid]); }
        const float inv = a.inv_in ? (tid < a.n ? a.inv_in[tid] : 0.0f) : rsqrtf(block_ss / float(a.k) + a.eps);
        inv_s[tid] = inv;
        if (a.inv_out && blockIdx.x == 0 && tid < a.n) a.inv_out[tid] = inv;
        x_up[tid] = 1.0f;
        x_down[tid] = 1.0f;
        if (INT8 && !(mx == 0.0f || (mx >= 0.015625f && mx < 32768.0f))) {
            const uint32_t ex = max((__float_as_uint(mx) >> 23) & 0xffu, 15u);  // mx in [2^(ex-127), 2^(ex-126))
            x_down[tid] = __uint_as_float((268u - ex) << 23);                   // puts it in [2^14, 2^15)
            x_up[tid] = __uint_as_float((ex - 14u) << 23);
            rescale_s = 1u;
        }
    }
    if (!INT8 && a.Xb && !st_mbar_wait(st_smem_u32(&bars[STREAM_MAX_STAGES]), 0) && lane == 0 && a.err_flag) atomicExch(a.err_flag, 2u);
    __syncthreads();
    if (INT8 && rescale_s) {  // (rare) once more from the source, scaled
        for (uint32_t i = tid; i < total; i += 512) {
            const uint32_t tk = i / n4, c = i % n4;
            uint32_t p0, p1;
            if (a.Xb) {
                const uint2 v = reinterpret_cast<const uint2*>(a.Xb + size_t(tk) * a.k)[c];
                p0 = v.x;
                p1 = v.y;
            } else {
                const float4 v = reinterpret_cast<const float4*>(a.X)[i];
                p0 = pack_bf16(v.x, v.y);
                p1 = pack_bf16(v.z, v.w);
            }
            put(tk, c, p0, p1, x_down[tk]);
        }
        __syncthreads();
    }

    if (tid == 0) SP_TIME(sp_t[2]);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint32_t buf = 0;
    const bool has_x = g < a.n;
    for (uint32_t item = 0; item < n_items; item++) {
        const uint32_t rt = blockIdx.x + (item / slices) * gridDim.x, sl = item % slices, st = item % n_stages, row0 = rt * 16;
        const uint32_t count = min(n_tiles - sl * 32, 32u);  // 64-byte tiles in this slice
        // One scale per row, applied once after the sum (from shared memory; past its room, asked for before the wait).
        float row_sl = 1.0f, row_sh = 1.0f;
        if (INT8 && !grouped && sl + 1 == slices && item / slices >= STREAM_SCALE_TILES) {
            row_sl = bf16_to_f32(a.scales[row0 + g]);
            row_sh = bf16_to_f32(a.scales[row0 + g + 8]);
        }
        // The residual this thread will add to (warps 0..3, see below): asked for now, there when the sums are.
        float resid = 0.0f;
        if (a.epi == EPI_RESID && sl + 1 == slices && tid < 128 && tid / 16 < a.n) resid = a.base[size_t(tid / 16) * a.m + row0 + tid % 16];
        if (!st_mbar_wait(st_smem_u32(&bars[st]), (item / n_stages) & 1) && lane == 0 && a.err_flag) atomicExch(a.err_flag, 2u);
        const uint8_t* sw = stages + size_t(st) * STREAM_STAGE;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t kt = warp + NW * u;  // tile within the slice
            if (kt >= count) break;             // (the same for the whole warp)
            const uint4 wl = *reinterpret_cast<const uint4*>(sw + g * STREAM_ROW + kt * 64 + t * 16);
            const uint4 wh = *reinterpret_cast<const uint4*>(sw + (g + 8) * STREAM_ROW + kt * 64 + t * 16);
            const uint32_t k0 = (sl * STREAM_SLICE + kt * 64 + t * 16) / WB;  // this lane's first weight of the tile
            uint32_t xb[E / 2];
            if (has_x) {
                const uint4* xp = reinterpret_cast<const uint4*>(xs + size_t(g) * xrs + size_t(k0) * 2);
#pragma unroll
                for (int q = 0; q < E / 8; q++) {
                    const uint4 v = xp[q];
                    xb[4 * q] = v.x; xb[4 * q + 1] = v.y; xb[4 * q + 2] = v.z; xb[4 * q + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < E / 2; q++) xb[q] = 0u;
            }
            uint32_t al[E / 2], ah[E / 2];  // rows g and g + 8 as bf16 pairs
            if (INT8) {
                cvt_i8x4_f16(wl.x, al[0], al[1]); cvt_i8x4_f16(wl.y, al[2], al[3]); cvt_i8x4_f16(wl.z, al[4], al[5]); cvt_i8x4_f16(wl.w, al[6], al[7]);
                cvt_i8x4_f16(wh.x, ah[0], ah[1]); cvt_i8x4_f16(wh.y, ah[2], ah[3]); cvt_i8x4_f16(wh.z, ah[4], ah[5]); cvt_i8x4_f16(wh.w, ah[6], ah[7]);
            } else {
                al[0] = wl.x; al[1] = wl.y; al[2] = wl.z; al[3] = wl.w;
                ah[0] = wh.x; ah[1] = wh.y; ah[2] = wh.z; ah[3] = wh.w;
            }
            if (grouped) {
                float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < KS; ks++) mma_f16(tmp, al[2 * ks], ah[2 * ks], al[2 * ks + 1], ah[2 * ks + 1], xb[2 * ks], xb[2 * ks + 1]);
                const uint32_t gi = k0 / a.group;
                const float sl_ = bf16_to_f32(a.scales[size_t(row0 + g) * ng + gi]);
                const float sh_ = bf16_to_f32(a.scales[size_t(row0 + g + 8) * ng + gi]);
                acc[0] += tmp[0] * sl_; acc[1] += tmp[1] * sl_; acc[2] += tmp[2] * sh_; acc[3] += tmp[3] * sh_;
            } else if (INT8) {
#pragma unroll
                for (int ks = 0; ks < KS; ks++) mma_f16(acc, al[2 * ks], ah[2 * ks], al[2 * ks + 1], ah[2 * ks + 1], xb[2 * ks], xb[2 * ks + 1]);
            } else {
#pragma unroll
                for (int ks = 0; ks < KS; ks++) mma_bf16(acc, al[2 * ks], ah[2 * ks], al[2 * ks + 1], ah[2 * ks + 1], xb[2 * ks], xb[2 * ks + 1]);
            }
        }
        if (sl + 1 == slices) {  // the row tile is complete: add up the warps and store
            if (INT8 && !grouped && item / slices < STREAM_SCALE_TILES) {
                row_sl = row_scale[(item / slices) * 16 + g];
                row_sh = row_scale[(item / slices) * 16 + g + 8];
            }
            acc[0] *= row_sl; acc[1] *= row_sl; acc[2] *= row_sh; acc[3] *= row_sh;
            float* rb = red + size_t(buf) * NW * 128 + warp * 128;  // [row][token]
            rb[g * 8 + 2 * t] = acc[0];
            rb[g * 8 + 2 * t + 1] = acc[1];
            rb[(g + 8) * 8 + 2 * t] = acc[2];
            rb[(g + 8) * 8 + 2 * t + 1] = acc[3];
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        }
        __syncthreads();  // every warp is done with the stage (and, after a row tile, has left its sums)
        if (warp == NW - 1 && item + n_stages < n_items) request(item + n_stages);
        if (warp == NW - 2 && item + n_stages + STREAM_AHEAD < n_items) prefetch(item + n_stages + STREAM_AHEAD);
        if (sl + 1 == slices) {
            // Warps 0..3: thread (token b, row r), consecutive threads on consecutive rows of one token. The buffer
            // alternates: a warp can be one row tile ahead of the four that are still adding up, never two.
            if (tid < 128) {
                const uint32_t r = tid % 16, b = tid / 16;
                const float* rp = red + size_t(buf) * NW * 128 + r * 8 + b;
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < NW; w++) sum += rp[w * 128];
                if (INT8) sum *= x_up[b];  // exact: a power of two
                const float partner = __shfl_down_sync(0xffffffffu, sum, 1);  // row r + 1 of the same token (r is even where it is used)
                if (b < a.n) {
                    const float inv = inv_s[b];
                    if (a.epi == EPI_SWIGLU) {
                        if (r % 2 == 0) store_swiglu(a, b, row0 + r, sum, partner, inv);
                    } else if (a.epi == EPI_QKV) {
                        if (r % 2 == 0) {  // qkv_store_pair with the token's table entries from shared memory
                            const uint32_t hd = a.q.kv.hd, row = row0 + r, head = row / hd, pair = (row % hd) / 2;
                            float y0 = sum * inv, y1 = partner * inv;
                            bool done = false;
                            if (head < a.q.n_heads + a.q.kv.n_kv) {
                                const float2 cs = q_cs[b][pair];
                                const float r0 = __fadd_rn(__fmul_rn(cs.x, y0), __fmul_rn(cs.y, y1));
                                const float r1 = __fsub_rn(__fmul_rn(cs.x, y1), __fmul_rn(cs.y, y0));
                                if (head < a.q.n_heads) {
                                    reinterpret_cast<uint32_t*>(a.q.q_b)[(size_t(a.t0 + b) * a.q.n_heads + head) * (hd / 2) + pair] =
                                        pack_bf16(__fmul_rn(r0, a.q.scale_log2), __fmul_rn(r1, a.q.scale_log2));
                                    done = true;
                                }
                                y0 = r0;
                                y1 = r1;
                            }
                            if (!done && q_kvrow[b] != ~size_t(0)) {
                                const bool is_v = head >= a.q.n_heads + a.q.kv.n_kv;
                                const uint32_t kvh = head - a.q.n_heads - (is_v ? a.q.kv.n_kv : 0);
                                const size_t at = q_kvrow[b] + size_t(kvh) * (size_t(1) << a.q.kv.page_shift) * hd;
                                reinterpret_cast<uint32_t*>((is_v ? a.q.v_cache : a.q.k_cache) + at)[pair] = pack_bf16(y0, y1);
                            }
                        }
                    } else if (a.epi == EPI_RESID) {
                        const size_t o = size_t(b) * a.m + row0 + r;
                        const float y = a.ra * resid + a.rb * (a.scale * sum);
                        a.Y[o] = y;
                        if (a.Yb) a.Yb[o] = f32_to_bf16(y);
                    } else {
                        store_out(a, b, row0 + r, sum, inv);
                    }
                }
            }
            buf ^= 1;
        }
    }
    if (tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
        SP_TIME(sp_t[3]);
        [[maybe_unused]] const unsigned tags[4] = {1, 2, 5, 3}, last[1] = {4};
        if (blockIdx.x == 0) SP_WRITE(sp_t, tags, 4);
        else SP_WRITE(sp_t + 3, last, 1);
    }
}

// Shared memory of the streamed kernel besides its stages: two buffers for the warps' sums and the staged activations.
static size_t stream_fixed_smem(const MatArgs& a) { return 2 * 16 * 128 * 4 + size_t(a.n) * (size_t(a.k) * 2 + 16); }

bool matmul_stream_fits(const MatArgs& a) {
    const bool grouped = a.int8 && a.group < a.k;
    const uint32_t row_bytes = a.k * (a.int8 ? 1 : 2);
    // (a scale group must cover whole 64-byte tiles: the four lanes of an mma row add up one tile's k)
    return !(a.n > 8 || row_bytes % 64 || a.m % 16 || (grouped && a.group % 64) || stream_fixed_smem(a) + 2 * STREAM_STAGE > STREAM_SMEM_MAX);
}

void launch_matmul_stream(const MatArgs& a, uint32_t sm_count, cudaStream_t s) {
    if (!matmul_stream_fits(a)) {
        if (a.epi == EPI_QKV) throw Error("internal: the qkv epilogue needs the streamed matmul's shapes");
        launch_matmul_rows(a, s);
        return;
    }
    static PerDevice configured;
    configured.once([] {
        VLT_CUDA(cudaFuncSetAttribute(matmul_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(STREAM_SMEM_MAX)));
        VLT_CUDA(cudaFuncSetAttribute(matmul_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(STREAM_SMEM_MAX)));
    });
    // Two resident blocks per SM with two or three stages each where shared memory allows (their row-tile meetings
    // then overlap), else one with up to six.
    const size_t fixed = stream_fixed_smem(a), half = 108 * 1024, whole = STREAM_SMEM_MAX;
    const uint32_t per_sm = fixed + 2 * STREAM_STAGE <= half ? 2 : 1;
    const uint32_t n_stages = uint32_t(std::min<size_t>(((per_sm == 2 ? half : whole) - fixed) / STREAM_STAGE, per_sm == 2 ? 3 : STREAM_MAX_STAGES));
    const uint32_t grid = std::min(a.m / 16, sm_count * per_sm);
    const size_t smem = fixed + size_t(n_stages) * STREAM_STAGE;
    if (a.int8) launch_pdl(matmul_stream_kernel<true>, grid, 512, smem, s, a, n_stages);
    else launch_pdl(matmul_stream_kernel<false>, grid, 512, smem, s, a, n_stages);
}

}  // namespace vlt
