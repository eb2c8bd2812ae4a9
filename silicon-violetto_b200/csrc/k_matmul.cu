// Matmuls for steps of at most 8 tokens: weights streamed once from HBM into registers and
// multiplied on the tensor cores (the reference's "stream" GEMM, kernels.metal:516-690, and its
// GEMV, :211-317), plus a scalar kernel for any shape (cross-check, odd scale groups).
//
// Y[t][row] = epilogue(W[row] . bf16(X[t])), W [m][k] row-major bf16 or int8 with bf16 scales
// per group of consecutive k, X fp32 [n][k]. 1/rms(X[t]) is accumulated in the same pass
// (kernels.metal:239-251,286), so a folded RMSNorm costs no extra kernel.
#include "kernels.h"

namespace vlt {

// kernels.metal:184-209 `epilogue`, `epilogue_swiglu`, for a plain decoder (scales and residual
// lambdas are 1, the head has no softcap).
__device__ __forceinline__ void store_out(const MatArgs& a, uint32_t t, uint32_t row, float acc, float inv) {
    const size_t o = size_t(t) * a.m + row;
    float y;
    switch (a.epi) {
    case EPI_NORM: y = acc * inv; break;
    case EPI_RESID: y = a.base[o] + acc; break;
    case EPI_HEAD: y = row < a.vocab_real ? acc * inv : -INFINITY; break;
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

// kernels.metal:749-801 `qkv_post` on one (even, odd) pair of rows of the qkv projection of token t: RoPE on q and k
// (interleaved pairs, the angle of the token's position), q scaled by scale * log2(e) and rounded to bf16 for the
// attention, k and v rounded to bf16 into the token's cache row (its run's first position + its row). Every float
// operation is a single rounded one, as in `qkv_post_kernel`, so both forms give the same bits.
__device__ __forceinline__ void qkv_store_pair(const QkvEpilogue& q, uint32_t t, uint32_t row, float y0, float y1) {
    const uint32_t hd = q.kv.hd, head = row / hd, pair = (row % hd) / 2;
    const uint32_t slot = q.meta[2 * t], pos = q.meta[2 * t + 1];
    if (head < q.n_heads + q.kv.n_kv) {
        const float2 cs = reinterpret_cast<const float2*>(q.rope)[size_t(pos) * (hd / 2) + pair];
        const float r0 = __fadd_rn(__fmul_rn(cs.x, y0), __fmul_rn(cs.y, y1));
        const float r1 = __fsub_rn(__fmul_rn(cs.x, y1), __fmul_rn(cs.y, y0));
        if (head < q.n_heads) {
            reinterpret_cast<uint32_t*>(q.q_b)[(size_t(t) * q.n_heads + head) * (hd / 2) + pair] = pack_bf16(__fmul_rn(r0, q.scale_log2), __fmul_rn(r1, q.scale_log2));
            return;
        }
        y0 = r0;
        y1 = r1;
    }
    const uint32_t run_row = q.tin[2 * t + 1];
    const uint32_t cpos = q.cpos ? q.cpos[t] : q.meta[2 * (t - run_row) + 1] + run_row;
    if (cpos == NO_TOK) return;  // (the drafter's passes leave out the rows that are not on the accepted path)
    const bool is_v = head >= q.n_heads + q.kv.n_kv;
    const size_t at = kv_row(q.kv, q.layer, q.page_table, slot, head - q.n_heads - (is_v ? q.kv.n_kv : 0), cpos);
    reinterpret_cast<uint32_t*>((is_v ? q.v_cache : q.k_cache) + at)[pair] = pack_bf16(y0, y1);
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

// A block takes 16 MT rows and all of k; its 16 warps take k tiles in turn and add up their
// sums through shared memory in warp order. Per tile a lane loads 16 bytes of row g and of row
// g + 8 of each m16 tile (g = lane / 4) and 16 or 8 floats of token g; since the contraction
// index may be permuted freely, lane t's consecutive k are used as k-slots (2t, 2t+1, 2t+8,
// 2t+9) of successive mma steps for A and B alike, so every load is contiguous.
template <bool INT8, int MT>
__global__ void __launch_bounds__(512) matmul_stream_kernel(MatArgs a) {
    pdl_start();
    constexpr int NW = 16;
    constexpr int E = INT8 ? 16 : 8;  // weights per 16-byte load
    constexpr int KT = 4 * E;         // k per tile
    constexpr int KS = E / 4;         // mma steps per tile
    __shared__ float red[NW][MT * 16][8];
    __shared__ float ss_red[NW][8];
    __shared__ float fin[MT * 16][8];
    __shared__ float inv_s[8];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * (16 * MT);
    const uint32_t n_tiles = a.k / KT;
    const bool grouped = INT8 && a.group < a.k;
    const uint32_t ng = INT8 ? a.k / a.group : 1;
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][i] = 0.0f;
    float ss = 0.0f;
    const bool has_x = g < a.n;
    const float* xrow = a.X + size_t(has_x ? g : 0) * a.k;

#pragma unroll(MT == 1 ? 4 : 2)  // loads in flight per lane: deep k (8 tiles a warp at k = 8192) would otherwise be four round trips
    for (uint32_t kt = warp; kt < n_tiles; kt += NW) {
        const uint32_t k0 = kt * KT + t * E;
        uint4 wl[MT], wh[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const size_t e = size_t(row0 + mt * 16 + g) * a.k + k0;
            const size_t bytes = INT8 ? 1 : 2;
            wl[mt] = __ldg(reinterpret_cast<const uint4*>(a.W + e * bytes));
            wh[mt] = __ldg(reinterpret_cast<const uint4*>(a.W + (e + size_t(8) * a.k) * bytes));
        }
        uint32_t xb[E / 2];
        if (has_x) {
#pragma unroll
            for (int j = 0; j < E / 4; j++) {
                const float4 v = *reinterpret_cast<const float4*>(xrow + k0 + 4 * j);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                xb[2 * j] = pack_bf16(v.x, v.y);
                xb[2 * j + 1] = pack_bf16(v.z, v.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < E / 2; j++) xb[j] = 0u;
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            uint32_t al[E / 2], ah[E / 2];  // rows g and g + 8 as bf16 pairs
            if (INT8) {
                cvt_i8x4(wl[mt].x, al[0], al[1]); cvt_i8x4(wl[mt].y, al[2], al[3]); cvt_i8x4(wl[mt].z, al[4], al[5]); cvt_i8x4(wl[mt].w, al[6], al[7]);
                cvt_i8x4(wh[mt].x, ah[0], ah[1]); cvt_i8x4(wh[mt].y, ah[2], ah[3]); cvt_i8x4(wh[mt].z, ah[4], ah[5]); cvt_i8x4(wh[mt].w, ah[6], ah[7]);
            } else {
                al[0] = wl[mt].x; al[1] = wl[mt].y; al[2] = wl[mt].z; al[3] = wl[mt].w;
                ah[0] = wh[mt].x; ah[1] = wh[mt].y; ah[2] = wh[mt].z; ah[3] = wh[mt].w;
            }
            if (grouped) {
                float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < KS; ks++) mma_bf16(tmp, al[2 * ks], ah[2 * ks], al[2 * ks + 1], ah[2 * ks + 1], xb[2 * ks], xb[2 * ks + 1]);
                const uint32_t gi = (kt * KT) / a.group;
                const float sl = bf16_to_f32(a.scales[size_t(row0 + mt * 16 + g) * ng + gi]);
                const float sh = bf16_to_f32(a.scales[size_t(row0 + mt * 16 + g + 8) * ng + gi]);
                acc[mt][0] += tmp[0] * sl; acc[mt][1] += tmp[1] * sl; acc[mt][2] += tmp[2] * sh; acc[mt][3] += tmp[3] * sh;
            } else {
#pragma unroll
                for (int ks = 0; ks < KS; ks++) mma_bf16(acc[mt], al[2 * ks], ah[2 * ks], al[2 * ks + 1], ah[2 * ks + 1], xb[2 * ks], xb[2 * ks + 1]);
            }
        }
    }
    // One scale per row: applied once, after the sum.
    if (INT8 && !grouped) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const float sl = bf16_to_f32(a.scales[row0 + mt * 16 + g]), sh = bf16_to_f32(a.scales[row0 + mt * 16 + g + 8]);
            acc[mt][0] *= sl; acc[mt][1] *= sl; acc[mt][2] *= sh; acc[mt][3] *= sh;
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        red[warp][mt * 16 + g][2 * t] = acc[mt][0];
        red[warp][mt * 16 + g][2 * t + 1] = acc[mt][1];
        red[warp][mt * 16 + g + 8][2 * t] = acc[mt][2];
        red[warp][mt * 16 + g + 8][2 * t + 1] = acc[mt][3];
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (t == 0) ss_red[warp][g] = ss;
    __syncthreads();
    const uint32_t tid = threadIdx.x;
    if (tid < MT * 16 * 8) {
        const uint32_t r = tid / 8, b = tid % 8;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++) s += red[w][r][b];
        fin[r][b] = s;
    }
    if (tid < 8) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++) s += ss_red[w][tid];
        const float inv = a.inv_in ? (tid < a.n ? a.inv_in[tid] : 0.0f) : rsqrtf(s / float(a.k) + a.eps);
        inv_s[tid] = inv;
        if (a.inv_out && blockIdx.x == 0 && tid < a.n) a.inv_out[tid] = inv;
    }
    __syncthreads();
    if (tid < MT * 16 * 8) {
        const uint32_t b = tid / (MT * 16), r = tid % (MT * 16);  // consecutive threads: consecutive rows of one token
        if (b < a.n) {
            if (a.epi == EPI_SWIGLU) {
                if (r % 2 == 0) store_swiglu(a, b, row0 + r, fin[r][b], fin[r + 1][b], inv_s[b]);
            } else if (a.epi == EPI_QKV) {
                if (r % 2 == 0) qkv_store_pair(a.q, a.t0 + b, row0 + r, fin[r][b] * inv_s[b], fin[r + 1][b] * inv_s[b]);
            } else {
                store_out(a, b, row0 + r, fin[r][b], inv_s[b]);
            }
        }
    }
}

bool matmul_stream_fits(const MatArgs& a) {
    const uint32_t kt = a.int8 ? 64 : 32;
    const bool grouped = a.int8 && a.group < a.k;
    return !(a.n > 8 || a.k % kt || a.m % 16 || (grouped && a.group % kt));
}

void launch_matmul_stream(const MatArgs& a, uint32_t sm_count, cudaStream_t s) {
    if (!matmul_stream_fits(a)) {
        if (a.epi == EPI_QKV) throw Error("internal: the qkv epilogue needs the streamed matmul's shapes");
        launch_matmul_rows(a, s);
        return;
    }
    // Rows per block: as many as still leave about two blocks per SM.
    int mt = 1;
    if (a.m % 32 == 0 && a.m / 32 >= 2 * sm_count) mt = 2;
    if (a.m % 64 == 0 && a.m / 64 >= 2 * sm_count) mt = 4;
    const uint32_t grid = a.m / (16 * mt);
#define VLT_STREAM(I8, MT) { launch_pdl(matmul_stream_kernel<I8, MT>, grid, 512, 0, s, a); }
    if (a.int8) {
        if (mt == 1) VLT_STREAM(true, 1) else if (mt == 2) VLT_STREAM(true, 2) else VLT_STREAM(true, 4)
    } else {
        if (mt == 1) VLT_STREAM(false, 1) else if (mt == 2) VLT_STREAM(false, 2) else VLT_STREAM(false, 4)
    }
#undef VLT_STREAM
}

}  // namespace vlt
