// Decode / verify attention over the paged KV cache on the tensor cores.
//
// The reference's attn_verify (kernels.metal:891-1167) reads a sequence's cached keys once for
// all rows of its run: the run's T <= 8 tokens x the G query heads of one kv head are packed into
// the MMA's query dimension (column p = G i + h, :896), the cached keys are split across
// threadgroups (:900), the run's own rows are attended under each token's visibility mask (:989),
// and each threadgroup writes a partial per (token, head, split) that a second kernel merges.
// This kernel keeps that decomposition and changes what B200 wants changed:
//   - K and V pages (16 tokens x 64 dims, 2 KiB each) come in by TMA into 128-byte-swizzled
//     shared memory, a four-stage ring per warp, and go to the MMAs through ldmatrix;
//   - the softmax keeps a running maximum (a plain decoder has no q/k norm to bound the
//     scores, kernels.metal:803-806), and partials carry (m, l, o[64]);
//   - the step's own rows are already in the cache (written by qkv_post), so they are read like
//     any other key and only the pages at or past the run's first position are masked.
// grid (kv heads, splits, tiles), 4 warps; warp w takes pages w, w + 4, ... of its split.
#include <cuda.h>

#include "kernels.h"

namespace vlt {

static constexpr int ATTN_WARPS = 4;
static constexpr int ATTN_STAGES = 3;
static constexpr uint32_t PAGE = 16, HD = 64;
static constexpr uint32_t STAGE_BYTES = 2 * PAGE * HD * 2;  // K then V
static constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// A bounded wait: false if the barrier did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = SPIN_LIMIT) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x),
                 "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MT: m16 tiles of query columns (T * G <= 16 MT).
template <int MT>
__global__ void __launch_bounds__(ATTN_WARPS * 32, 4) attn_mma_kernel(AttnArgs a, const __grid_constant__ AttnMaps maps) {
    pdl_start();
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4..9.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bars[ATTN_WARPS][ATTN_STAGES];
    __shared__ __align__(128) uint4 qs[MT * 16 * 8];  // 128-byte aligned: fragment addresses below differ by an XOR of address bits 5..6

    const uint32_t kvh = blockIdx.x, split = blockIdx.y, tile = blockIdx.z;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const uint32_t G = a.n_heads / a.kv.n_kv;
    const uint32_t t0 = a.tiles[2 * tile], T = a.tiles[2 * tile + 1];
    const uint32_t slot = a.meta[2 * t0], p0 = a.meta[2 * t0 + 1];
    const uint32_t n_keys = p0 + T, n_cols = T * G;
    const uint32_t k_begin = split * a.keys_per_split;
    const uint32_t k_end = min(k_begin + a.keys_per_split, n_keys);

    auto part_of = [&](uint32_t p) {  // column p's partial for this split
        return a.part + ((size_t(t0 + p / G) * a.n_heads + kvh * G + p % G) * a.max_splits + split) * ATTN_PART;
    };
    if (k_begin >= n_keys) {  // nothing for this split: the merge skips m = -inf
        for (uint32_t p = threadIdx.x; p < n_cols; p += blockDim.x) {
            float* pp = part_of(p);
            pp[0] = -INFINITY;
            pp[1] = 0.0f;
        }
        return;
    }

    // This warp's pages: page_begin + warp, + ATTN_WARPS, ...
    const uint32_t page_begin = k_begin / PAGE, page_end = (k_end + PAGE - 1) / PAGE;
    const uint32_t my_pages = page_begin + warp < page_end ? (page_end - page_begin - warp + ATTN_WARPS - 1) / ATTN_WARPS : 0;
    uint8_t* wbuf = smem + size_t(warp) * ATTN_STAGES * STAGE_BYTES;
    const uint32_t* ptab = a.page_table + size_t(slot) * a.kv.max_pages;
    const uint32_t row_base = a.layer * a.kv.n_pages;  // in pages

    // Page ids are fetched 32 at a time (lane j holds the id of this warp's page 32 b + j), a batch
    // ahead, so that no TMA issue waits on a page-table load.
    auto load_ids = [&](uint32_t batch) {
        const uint32_t i = batch * 32 + lane;
        return i < my_pages ? ptab[page_begin + warp + i * ATTN_WARPS] : 0u;
    };
    uint32_t ids0 = load_ids(0), ids1 = load_ids(1), cur_batch = 0;

    // Q (bf16, RoPE and the softmax scale already applied) into shared memory as [row p][64 dims],
    // 16-byte chunks XOR-swizzled by the row; row p = G i + h is token i, head h of this kv head.
    {
        const uint4* qg = reinterpret_cast<const uint4*>(a.q_b);
        for (uint32_t c = threadIdx.x; c < MT * 16 * 8; c += ATTN_WARPS * 32) {
            const uint32_t p = c / 8, chunk = c % 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (p < n_cols) v = qg[(size_t(t0 + p / G) * a.n_heads + kvh * G + p % G) * 8 + chunk];
            qs[p * 8 + (chunk ^ (p & 7))] = v;
        }
    }
    if (threadIdx.x == 0) {
        for (int w = 0; w < ATTN_WARPS; w++)
            for (int s = 0; s < ATTN_STAGES; s++) mbar_init(smem_u32(&bars[w][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](uint32_t i) {  // all lanes: page i of this warp into stage i % STAGES
        if (i / 32 > cur_batch) {
            ids0 = ids1;
            cur_batch++;
            ids1 = load_ids(cur_batch + 1);
        }
        const uint32_t pg = __shfl_sync(0xffffffffu, ids0, i % 32);
        if (lane == 0) {
            const int y = int(((row_base + pg) * a.kv.n_kv + kvh) * PAGE);
            const uint32_t st = i % ATTN_STAGES, bar = smem_u32(&bars[warp][st]), dst = smem_u32(wbuf + st * STAGE_BYTES);
            mbar_expect_tx(bar, STAGE_BYTES);
            tma_load_2d(dst, &maps.k, 0, y, bar);
            tma_load_2d(dst + PAGE * HD * 2, &maps.v, 0, y, bar);
        }
    };
    for (uint32_t i = 0; i < min(my_pages, uint32_t(ATTN_STAGES)); i++) issue(i);

    // Q as A operands (a0: rows g, dims lo; a1: rows g + 8, lo; a2: g, hi; a3: g + 8, hi) are read from
    // shared memory for every page (keeping the 8 MT fragments in registers would cost a block per SM), and
    // the visibility masks of this lane's rows g and g + 8 stay in registers.
    const uint32_t lm = lane >> 3, lr = lane & 7;  // ldmatrix: lane -> (matrix, row)
    uint32_t q_addr[MT];  // fragment (mt, ks) is at q_addr[mt] ^ (ks << 5): the swizzle is an XOR of the 16-byte chunk index
    uint32_t vmask[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const uint32_t p = mt * 16 + 8 * (lm & 1) + lr;
        q_addr[mt] = smem_u32(&qs[p * 8 + ((lm >> 1) ^ (p & 7))]);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const uint32_t pr = mt * 16 + g + 8 * half;
            vmask[mt][half] = pr < n_cols ? a.vis[t0 + pr / G] : 0xffffffffu;
        }
    }

    float oacc[MT][8][4];
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
        for (int dn = 0; dn < 8; dn++)
#pragma unroll
            for (int i = 0; i < 4; i++) oacc[mt][dn][i] = 0.0f;
        m_run[mt][0] = m_run[mt][1] = -INFINITY;
        l_run[mt][0] = l_run[mt][1] = 0.0f;
    }

    // This lane's ldmatrix row within a page (stages are 1024-byte aligned, rows 128 bytes: the swizzled
    // 16-byte chunk index is address bits 4..6, so the k step / dim pair is an XOR away).
    const uint32_t k_off = (8 * (lm >> 1) + lr) * 128 + (((lm & 1) ^ lr) << 4);
    const uint32_t v_off = (8 * (lm & 1) + lr) * 128 + (((lm >> 1) ^ lr) << 4);
    bool failed = false;
    for (uint32_t i = 0; i < my_pages; i++) {
        const uint32_t st = i % ATTN_STAGES, parity = (i / ATTN_STAGES) & 1;
        if (!mbar_wait(smem_u32(&bars[warp][st]), parity)) { failed = true; break; }
        const uint32_t kbase = smem_u32(wbuf + st * STAGE_BYTES), vbase = kbase + PAGE * HD * 2;
        const uint32_t key0 = (page_begin + warp + i * ATTN_WARPS) * PAGE;

        // S = Q K^T: n-tile nt = keys 8 nt .. 8 nt + 7 of the page.
        float sacc[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sacc[mt][nt][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t kb[4];  // b0, b1 of nt 0, then of nt 1
            ldmatrix_x4(kb, (kbase + k_off) ^ (uint32_t(ks) << 5));  // chunk 2 ks + (lm & 1), swizzled: an XOR of address bits 5..6
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                uint32_t qf[4];
                ldmatrix_x4(qf, q_addr[mt] ^ (uint32_t(ks) << 5));
                mma16816(sacc[mt][0], qf, kb[0], kb[1]);
                mma16816(sacc[mt][1], qf, kb[2], kb[3]);
            }
        }
        // Visibility: keys below p0 are seen by every row; key p0 + j by the rows whose mask has
        // bit j; keys from p0 + T on by none.
        if (key0 + PAGE > p0) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const uint32_t key = key0 + 8 * nt + 2 * t + (e & 1);
                        const uint32_t mask = vmask[mt][e >> 1];
                        const bool seen = key < p0 || (key < n_keys && ((mask >> (key - p0)) & 1u));
                        if (!seen) sacc[mt][nt][e] = -INFINITY;
                    }
        }
        // Online softmax; a row's statistics are shared by the four lanes of its quad.
        uint32_t pa[MT][4];
        float corr[MT][2];
        bool rescale = false;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float mx = fmaxf(fmaxf(sacc[mt][0][2 * half], sacc[mt][0][2 * half + 1]), fmaxf(sacc[mt][1][2 * half], sacc[mt][1][2 * half + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[mt][half], mx);
                const float m_use = m_new == -INFINITY ? 0.0f : m_new;
                corr[mt][half] = fast_exp2(m_run[mt][half] - m_use);
                rescale = rescale || corr[mt][half] != 1.0f;
                m_run[mt][half] = m_new;
                const float p00 = fast_exp2(sacc[mt][0][2 * half] - m_use), p01 = fast_exp2(sacc[mt][0][2 * half + 1] - m_use);
                const float p10 = fast_exp2(sacc[mt][1][2 * half] - m_use), p11 = fast_exp2(sacc[mt][1][2 * half + 1] - m_use);
                l_run[mt][half] = l_run[mt][half] * corr[mt][half] + (p00 + p01 + p10 + p11);
                pa[mt][half] = pack_bf16(p00, p01);      // a0 / a1: keys 2t, 2t + 1
                pa[mt][half + 2] = pack_bf16(p10, p11);  // a2 / a3: keys 8 + 2t, 9 + 2t
            }
        }
        if (__any_sync(0xffffffffu, rescale)) {  // a maximum moved somewhere in the warp: rare after the first pages
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int dn = 0; dn < 8; dn++) {
                    oacc[mt][dn][0] *= corr[mt][0];
                    oacc[mt][dn][1] *= corr[mt][0];
                    oacc[mt][dn][2] *= corr[mt][1];
                    oacc[mt][dn][3] *= corr[mt][1];
                }
        }
        // O += P V: n-tile dn = dims 8 dn .. 8 dn + 7.
#pragma unroll
        for (int dp = 0; dp < 4; dp++) {
            uint32_t vb[4];  // b0, b1 of dn = 2 dp, then of dn = 2 dp + 1
            ldmatrix_x4_trans(vb, (vbase + v_off) ^ (uint32_t(dp) << 5));  // chunk 2 dp + (lm >> 1), swizzled
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                mma16816(oacc[mt][2 * dp], pa[mt], vb[0], vb[1]);
                mma16816(oacc[mt][2 * dp + 1], pa[mt], vb[2], vb[3]);
            }
        }
        __syncwarp();
        if (i + ATTN_STAGES < my_pages) issue(i + ATTN_STAGES);
    }
    if (failed) {
        // A copy never arrived: say so, give the other copies in flight a bounded time, and leave.
        if (lane == 0) {
            atomicExch(a.err_flag, 1u);
            for (int s = 0; s < ATTN_STAGES; s++) mbar_wait(smem_u32(&bars[warp][s]), 0, 1u << 16);
        }
        return;
    }

    // Merge the four warps through shared memory (the stage ring is free now): every warp scales
    // its rows to the block's maximum, the block adds them up and writes the partial.
    __syncthreads();
    constexpr int ROWS = MT * 16, OS = HD + 8;        // the row stride keeps the float2 stores off each other's banks
    float* ms = reinterpret_cast<float*>(smem);      // [warp][row]
    float* ls = ms + ATTN_WARPS * ROWS;              // [warp][row], scaled
    float* os = ls + ATTN_WARPS * ROWS;              // [warp][row][OS], scaled
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int half = 0; half < 2; half++)
            if (t == 0) ms[warp * ROWS + mt * 16 + g + 8 * half] = m_run[mt][half];
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const uint32_t row = mt * 16 + g + 8 * half;
            float mm = ms[row];
#pragma unroll
            for (int w = 1; w < ATTN_WARPS; w++) mm = fmaxf(mm, ms[w * ROWS + row]);
            const float wgt = m_run[mt][half] == -INFINITY ? 0.0f : fast_exp2(m_run[mt][half] - mm);
            float l = l_run[mt][half];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (t == 0) ls[warp * ROWS + row] = l * wgt;
#pragma unroll
            for (int dn = 0; dn < 8; dn++)
                *reinterpret_cast<float2*>(os + (size_t(warp) * ROWS + row) * OS + 8 * dn + 2 * t) =
                    make_float2(oacc[mt][dn][2 * half] * wgt, oacc[mt][dn][2 * half + 1] * wgt);
        }
    }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < n_cols * HD; idx += blockDim.x) {
        const uint32_t p = idx / HD, d = idx % HD;
        float oo = 0.0f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; w++) oo += os[(size_t(w) * ROWS + p) * OS + d];
        float* pp = part_of(p);
        if (d == 0) {
            float mm = ms[p], ll = 0.0f;
#pragma unroll
            for (int w = 1; w < ATTN_WARPS; w++) mm = fmaxf(mm, ms[w * ROWS + p]);
#pragma unroll
            for (int w = 0; w < ATTN_WARPS; w++) ll += ls[w * ROWS + p];
            pp[0] = mm;
            pp[1] = ll;
        }
        pp[4 + d] = oo;
    }
}

// A 2-D tensor [rows][inner] with a box of [box_rows][box_inner], optionally 128- or 64-byte swizzled.
struct TmaEncoder {
    typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    Fn fn = nullptr;
    TmaEncoder() {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
            throw Error("cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<Fn>(p);
    }
};

void make_tensor_map_2d(void* out_map, const void* base, uint64_t inner, uint64_t rows, uint32_t box_inner, uint32_t box_rows, uint32_t elem_bytes,
                        bool swizzle128, bool swizzle64) {
    static TmaEncoder enc;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {inner * elem_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const CUresult r = enc.fn(static_cast<CUtensorMap*>(out_map), dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
}

// The K and V pools as [all layers' rows][64] bf16, a box of one page.
void attn_maps_init(AttnMaps* m, const uint16_t* k_cache, const uint16_t* v_cache, uint64_t total_rows) {
    static_assert(sizeof(CUtensorMap) == sizeof(m->k), "tensor map size");
    make_tensor_map_2d(&m->k, k_cache, HD, total_rows, HD, PAGE, 2, true);
    make_tensor_map_2d(&m->v, v_cache, HD, total_rows, HD, PAGE, 2, true);
}

void launch_attn_mma(const AttnArgs& a, cudaStream_t s) {
    const uint32_t G = a.n_heads / a.kv.n_kv;
    const size_t smem = size_t(ATTN_WARPS) * ATTN_STAGES * STAGE_BYTES + 1024;
    // kv heads fastest: the blocks that start together read neighbouring 2 KiB slabs of the same pages.
    const dim3 grid(a.kv.n_kv, a.max_splits, a.n_tiles);
    static bool configured = false;
    if (!configured) {
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured = true;
    }
    if (VERIFY_T * G <= 16) launch_pdl(attn_mma_kernel<1>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
    else launch_pdl(attn_mma_kernel<2>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
}

}  // namespace vlt
