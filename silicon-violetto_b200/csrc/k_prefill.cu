// Chunk (prefill) attention over the paged KV cache: the reference's attn_mma + attn_sum_reduce
// (kernels.metal:1169-1312; engine/src/engine/encode.rs:299-355 runs them whenever a step holds a run longer than
// 8 tokens) for steps that carry prompt chunks.
//
// The decode kernel (k_attn.cu) packs a run's <= 8 rows x G heads into the MMA's narrow side and streams the keys once
// per 8 rows: right when the keys dominate, wasteful for a chunk of hundreds of rows, whose every 8 rows would read the
// context again. Here the queries are the MMA's M side: a block owns 64 rows of one run and one query head (4 warps x
// 16 rows), walks the keys in blocks of 64 (four pages of K and of V by TMA into a three-stage ring of 128-byte-swizzled
// shared memory, shared by the four warps; the G heads of a kv head find the same pages in L2), and keeps the whole
// softmax online in registers: S = Q K^T lands in the accumulator layout that is the A-fragment layout of the next
// product, so P goes into O += P V without leaving the registers. No key split (a chunk has rows enough to fill the
// GPU), so no partials and no merge kernel: the block writes the normalised rows, fp32 and bf16.
//
// The step's own rows are in the cache already (the qkv projection's epilogue wrote them), so every key is read from
// there; what a row may see is the decode kernel's rule, per row: every cached key below the first position of its
// 8-row tile, and of that tile's keys those its `vis` mask names (causal for a chunk, the tree's for a verify run that
// shares the step). q arrives rotated, scaled by scale * log2(e) and rounded to bf16.
// Every mbarrier wait is bounded and sets the error word on time-out.
#include <cuda.h>

#include "kernels.h"
#include "mma.cuh"

namespace vlt {

namespace prefill {

constexpr uint32_t CQ = 64, CK = 64, HD = 64, PAGE = 16, WARPS = 4, STAGES = 3;
constexpr uint32_t STAGE_BYTES = 2 * CK * HD * 2;  // K block then V block
constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = SPIN_LIMIT) {
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x),
                 "r"(y), "r"(bar)
                 : "memory");
}
// grid (chunk tiles, query heads), 128 threads.
__global__ void __launch_bounds__(WARPS * 32) attn_chunk_kernel(ChunkAttnArgs a, const __grid_constant__ AttnMaps maps) {
    pdl_start();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));  // the swizzle is a function of address bits 4..9
    __shared__ uint64_t bars[STAGES];
    __shared__ uint32_t fail;

    const uint32_t tile = blockIdx.x, h = blockIdx.y, kvh = h / (a.n_heads / a.kv.n_kv);
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane >> 2, tq = lane & 3;
    const uint32_t t0 = a.ctiles[2 * tile], rows = a.ctiles[2 * tile + 1];
    const uint32_t slot = a.meta[2 * t0];

    // This thread's two rows (g and g + 8 of its warp's 16): the token, the first position of its 8-row tile and its mask.
    uint32_t tok[2], p8[2], vmask[2];
    bool live[2];
    uint32_t my_end = 0;  // one past the last key either row may see
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint32_t row = warp * 16 + g + 8 * r;
        live[r] = row < rows;
        tok[r] = t0 + (live[r] ? row : 0);
        const uint32_t in_run = a.tin[2 * tok[r] + 1];
        p8[r] = a.meta[2 * (tok[r] - in_run % 8) + 1];  // that token is the first of the 8-row tile: its position is the tile's
        vmask[r] = live[r] ? a.vis[tok[r]] : 0u;
        if (live[r] && vmask[r]) my_end = max(my_end, p8[r] + 32 - __clz(vmask[r]));
    }
    // The block walks keys [0, block_end): the furthest any of its rows sees.
    uint32_t block_end = my_end;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) block_end = max(block_end, __shfl_xor_sync(0xffffffffu, block_end, o));
    __shared__ uint32_t ends[WARPS];
    if (lane == 0) ends[warp] = block_end;
    if (tid == 0) {
        for (uint32_t s = 0; s < STAGES; s++) mbar_init(smem_u32(&bars[s]), 1);
        fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const uint32_t warp_end = ends[warp];
    block_end = max(max(ends[0], ends[1]), max(ends[2], ends[3]));
    const uint32_t n_blocks = (block_end + CK - 1) / CK;

    const uint32_t* ptab = a.page_table + size_t(slot) * a.kv.max_pages;
    const uint32_t row_base = a.layer * a.kv.n_pages;
    auto issue = [&](uint32_t b) {  // thread 0: key block b into stage b % STAGES
        const uint32_t st = b % STAGES, bar = smem_u32(&bars[st]), dst = smem_u32(smem + st * STAGE_BYTES);
        mbar_expect_tx(bar, STAGE_BYTES);
        for (uint32_t pi = 0; pi < CK / PAGE; pi++) {
            // Pages past the sequence's last hold nothing this block may see (masked below): any valid page will do.
            const uint32_t idx = min(b * (CK / PAGE) + pi, a.kv.max_pages - 1);
            const uint32_t pg = min(ptab[idx], a.kv.n_pages - 1);
            const int y = int(((row_base + pg) * a.kv.n_kv + kvh) * PAGE);
            tma_load_2d(dst + pi * PAGE * HD * 2, &maps.k, 0, y, bar);
            tma_load_2d(dst + CK * HD * 2 + pi * PAGE * HD * 2, &maps.v, 0, y, bar);
        }
    };
    if (tid == 0)
        for (uint32_t b = 0; b < min(n_blocks, STAGES); b++) issue(b);

    // Q fragments (A operands) straight from global memory: row g / g + 8, dims 16 ks + 2 tq (+ 8).
    uint32_t qa[4][4];
    {
        const uint32_t* q32 = reinterpret_cast<const uint32_t*>(a.q_b);
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const size_t r0 = (size_t(tok[0]) * a.n_heads + h) * (HD / 2) + 8 * ks + tq, r1 = (size_t(tok[1]) * a.n_heads + h) * (HD / 2) + 8 * ks + tq;
            qa[ks][0] = live[0] ? q32[r0] : 0u;
            qa[ks][1] = live[1] ? q32[r1] : 0u;
            qa[ks][2] = live[0] ? q32[r0 + 4] : 0u;
            qa[ks][3] = live[1] ? q32[r1 + 4] : 0u;
        }
    }
    // ldmatrix lane roles: matrix lm = lane / 8, row lr = lane % 8. A page is 16 rows of 128 bytes, 2 KiB (1024-byte aligned
    // halves), so the swizzled 16-byte chunk is (chunk ^ (row & 7)).
    const uint32_t lm = lane >> 3, lr = lane & 7;

    float oacc[8][4];  // O: n-tile jd = dims 8 jd .. 8 jd + 7; [0,1] row g, [2,3] row g + 8
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
#pragma unroll
    for (int jd = 0; jd < 8; jd++)
#pragma unroll
        for (int e = 0; e < 4; e++) oacc[jd][e] = 0.0f;

    bool failed = false;
    for (uint32_t b = 0; b < n_blocks; b++) {
        const uint32_t st = b % STAGES, parity = (b / STAGES) & 1;
        if (!mbar_wait(smem_u32(&bars[st]), parity)) { failed = true; }
        if (__any_sync(0xffffffffu, failed)) { if (lane == 0) fail = 1; }
        const uint32_t kbase = smem_u32(smem + st * STAGE_BYTES), vbase = kbase + CK * HD * 2, key0 = b * CK;
        if (!failed && key0 < warp_end) {  // (a warp whose rows see nothing of this block skips the arithmetic, not the barriers)
            // S = Q K^T: 16 rows x 64 keys; n-tile j = keys 8 j .. 8 j + 7.
            float sacc[8][4];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.0f;
                const uint32_t krow = 8 * j + lr, kaddr = kbase + (krow / PAGE) * (PAGE * HD * 2) + (krow % PAGE) * 128;
#pragma unroll
                for (int kp = 0; kp < 2; kp++) {  // k steps 2 kp and 2 kp + 1: chunks 4 kp + lm
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kaddr + (((4 * kp + lm) ^ (krow & 7)) << 4));
                    mma16816(sacc[j], qa[2 * kp], kb[0], kb[1]);
                    mma16816(sacc[j], qa[2 * kp + 1], kb[2], kb[3]);
                }
            }
            // What each row may see: keys below its tile's first position, and of the tile's keys those its mask names.
            const uint32_t lo = min(p8[0], p8[1]);
            if (key0 + CK > lo || !live[0] || !live[1]) {
#pragma unroll
                for (int j = 0; j < 8; j++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const uint32_t r = e >> 1, key = key0 + 8 * j + 2 * tq + (e & 1);
                        const bool seen = live[r] && (key < p8[r] || (key - p8[r] < 32 && ((vmask[r] >> (key - p8[r])) & 1u)));
                        if (!seen) sacc[j][e] = -INFINITY;
                    }
            }
            // Online softmax: a row's 64 scores sit in the four lanes of its quad.
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; j++) mx = fmaxf(mx, fmaxf(sacc[j][2 * r], sacc[j][2 * r + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[r], mx), m_use = m_new == -INFINITY ? 0.0f : m_new;
                corr[r] = fast_exp2(m_run[r] - m_use);
                m_run[r] = m_new;
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    sacc[j][2 * r] = fast_exp2(sacc[j][2 * r] - m_use);
                    sacc[j][2 * r + 1] = fast_exp2(sacc[j][2 * r + 1] - m_use);
                    sum += sacc[j][2 * r] + sacc[j][2 * r + 1];
                }
                l_run[r] = l_run[r] * corr[r] + sum;  // this lane's share of the row; the quad's shares meet at the end
            }
#pragma unroll
            for (int jd = 0; jd < 8; jd++) {
                oacc[jd][0] *= corr[0];
                oacc[jd][1] *= corr[0];
                oacc[jd][2] *= corr[1];
                oacc[jd][3] *= corr[1];
            }
            // O += P V: key step kk = keys 16 kk .. 16 kk + 15 (one page); P's accumulators are the A fragments.
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                uint32_t pa[4];
                pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
                pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
                pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
                pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
                const uint32_t vrow = 8 * (lm & 1) + lr, vaddr = vbase + kk * (PAGE * HD * 2) + vrow * 128;
#pragma unroll
                for (int dp = 0; dp < 4; dp++) {  // dims 16 dp .. 16 dp + 15: n-tiles 2 dp and 2 dp + 1
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vaddr + (((2 * dp + (lm >> 1)) ^ (vrow & 7)) << 4));
                    mma16816(oacc[2 * dp], pa, vb[0], vb[1]);
                    mma16816(oacc[2 * dp + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage
        if (fail) break;
        if (tid == 0 && b + STAGES < n_blocks) issue(b + STAGES);
    }
    if (fail) {
        // A copy never arrived: say so, give the copies in flight a bounded time, and leave.
        if (tid == 0) {
            atomicExch(a.err_flag, 3u);
            for (uint32_t s = 0; s < STAGES; s++) mbar_wait(smem_u32(&bars[s]), 0, 1u << 16);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!live[r]) continue;
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const size_t at = size_t(tok[r]) * a.n_heads * HD + h * HD;
#pragma unroll
        for (int jd = 0; jd < 8; jd++) {
            const float x = oacc[jd][2 * r] * inv, y = oacc[jd][2 * r + 1] * inv;
            *reinterpret_cast<float2*>(a.out + at + 8 * jd + 2 * tq) = make_float2(x, y);
            if (a.out_b) *reinterpret_cast<uint32_t*>(a.out_b + at + 8 * jd + 2 * tq) = pack_bf16(x, y);
        }
    }
}

}  // namespace prefill

void launch_attn_chunk(const ChunkAttnArgs& a, cudaStream_t s) {
    if (!a.n_ctiles) return;
    const size_t smem = size_t(prefill::STAGES) * prefill::STAGE_BYTES + 1024;
    static PerDevice configured;
    configured.once([smem] { VLT_CUDA(cudaFuncSetAttribute(prefill::attn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); });
    launch_pdl(prefill::attn_chunk_kernel, dim3(a.n_ctiles, a.n_heads), prefill::WARPS * 32, smem, s, a, *a.maps);
}

}  // namespace vlt
