// Decode / verify attention over the paged KV cache on the tensor cores.
//
// The reference's attn_verify (kernels.metal:891-1167) reads a sequence's cached keys once for
// all rows of its run: the run's T <= 8 tokens x the G query heads of one kv head are packed into
// the MMA's query dimension (column p = G i + h, :896), the cached keys are split across
// threadgroups (:900), the run's own rows are attended under each token's visibility mask (:989),
// and each threadgroup writes a partial per (token, head, split) that a second kernel merges.
// This kernel keeps that decomposition and changes what B200 wants changed:
//   - K and V pages (16 tokens x 64 dims, 2 KiB each) come in by TMA into 128-byte-swizzled
//     shared memory, a three-stage ring per warp, and go to the MMAs through ldmatrix;
//   - the softmax keeps a running maximum (a plain decoder has no q/k norm to bound the
//     scores, kernels.metal:803-806), and partials carry (m, l, o[64]);
//   - the step's own rows are already in the cache (written by the qkv projection's epilogue or qkv_post), so they are read like
//     any other key and only the pages at or past the run's first position are masked.
// grid (kv heads, splits, tiles), 4 warps; warp w takes pages w, w + 4, ... of its split.
#include <cuda.h>

#include <algorithm>

#include "kernels.h"
#include "mma.cuh"

namespace vlt {

static constexpr int ATTN_WARPS = 4;
static constexpr int ATTN_STAGES = 3;
static constexpr uint32_t PAGE = 16, HD = 64;
static constexpr uint32_t STAGE_BYTES = 2 * PAGE * HD * 2;  // K then V
static constexpr uint32_t SPIN_LIMIT = 1u << 24;

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
// NT: n8 tiles of query columns (column p = G i + h is token i, head h of this kv head; T * G <= 8 NT).
// The keys are the MMAs' M side: S^T = K Q^T per page (16 keys x 8 NT columns), O^T += V^T P^T
// (64 dims x 8 NT columns), so a page costs 8 NT MMAs whatever the number of query rows, the
// statistics of a column live in the lanes that hold it, and P^T reaches the second MMA through
// movmatrix. ATTN_CTAS blocks of 4 warps per SM.
template <int NT>
__global__ void __launch_bounds__(ATTN_WARPS * 32, NT <= 3 ? 4 : 3) attn_mma_kernel(AttnArgs a, const __grid_constant__ AttnMaps maps) {
    pdl_start();
    constexpr int NTP = (NT + 1) / 2 * 2, NC = 8 * NT;  // q rows in shared memory: whole ldmatrix.x4 pairs of n-tiles
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 4..9.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bars[ATTN_WARPS][ATTN_STAGES];
    __shared__ __align__(128) uint4 qs[NTP * 8 * 8];  // 128-byte aligned: fragment addresses below differ by an XOR of address bits 5..6

    const uint32_t kvh = blockIdx.x, split = blockIdx.y, tile = blockIdx.z;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const uint32_t G = a.n_heads / a.kv.n_kv;
    const uint32_t t0 = a.tiles[2 * tile], T = a.tiles[2 * tile + 1];
    const uint32_t slot = a.meta[2 * t0], p0 = a.meta[2 * t0 + 1];
    const uint32_t n_keys = p0 + T, n_cols = min(T * G, uint32_t(NC));
    // A windowed layer starts at the page that holds the first key of the tile's last `window`.
    const uint32_t k_lo = a.window && n_keys > a.window ? (n_keys - a.window) / PAGE * PAGE : 0;
    const uint32_t k_begin = k_lo + split * a.keys_per_split;
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

    // Q (bf16, RoPE and the softmax scale already applied) into shared memory as [column p][64 dims],
    // 16-byte chunks XOR-swizzled by the row.
    {
        const uint4* qg = reinterpret_cast<const uint4*>(a.q_b);
        for (uint32_t c = threadIdx.x; c < NTP * 8 * 8; c += ATTN_WARPS * 32) {
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

    // ldmatrix lane roles: lane -> (matrix lm, row lr). Rows are 128 bytes and tiles 1024-byte aligned, so the
    // swizzled 16-byte chunk index is address bits 4..6 and a k step / dim pair is an XOR of bits 5..6 away.
    const uint32_t lm = lane >> 3, lr = lane & 7;
    // K as A (keys x dims, straight) and V^T as A (dims x keys, .trans): key 8 (lm & 1) + lr / 8 (lm >> 1) + lr.
    const uint32_t k_off = (8 * (lm & 1) + lr) * 128 + (((lm >> 1) ^ lr) << 4);
    const uint32_t v_off = (8 * (lm >> 1) + lr) * 128 + (((lm & 1) ^ lr) << 4);
    // Q^T as B: n-tile pair jp covers columns 16 jp ..; matrix lm -> n-tile 2 jp + (lm >> 1), chunk 2 ks + (lm & 1).
    const uint32_t q_off = smem_u32(qs) + (8 * (lm >> 1) + lr) * 128 + (((lm & 1) ^ lr) << 4);

    // This lane's columns: 8 j + 2 t and 8 j + 2 t + 1 of every n-tile j; their visibility masks.
    uint32_t vmask[NT][2];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t p = 8 * j + 2 * t + e;
            vmask[j][e] = p < n_cols ? a.vis[t0 + p / G] : 0xffffffffu;
        }

    float oacc[4][NT][4];  // O^T: [dims 16 dm + g (+ 8)][columns 8 j + 2 t (+ 1)]
    float m_run[NT][2], l_run[NT][2];  // per column; l is this lane's share (its keys g and g + 8)
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
        for (int dm = 0; dm < 4; dm++)
#pragma unroll
            for (int e = 0; e < 4; e++) oacc[dm][j][e] = 0.0f;
        m_run[j][0] = m_run[j][1] = -INFINITY;
        l_run[j][0] = l_run[j][1] = 0.0f;
    }

    bool failed = false;
    for (uint32_t i = 0; i < my_pages; i++) {
        const uint32_t st = i % ATTN_STAGES, parity = (i / ATTN_STAGES) & 1;
        if (!mbar_wait(smem_u32(&bars[warp][st]), parity)) { failed = true; break; }
        const uint32_t kbase = smem_u32(wbuf + st * STAGE_BYTES), vbase = kbase + PAGE * HD * 2;
        const uint32_t key0 = (page_begin + warp + i * ATTN_WARPS) * PAGE;

        // S^T = K Q^T: rows = the page's keys g and g + 8, columns = this lane's.
        float sacc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) sacc[j][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t ka[4];
            ldmatrix_x4(ka, (kbase + k_off) ^ (uint32_t(ks) << 5));
#pragma unroll
            for (int jp = 0; jp < NTP / 2; jp++) {
                uint32_t qb[4];  // b0, b1 of n-tile 2 jp, then of 2 jp + 1
                ldmatrix_x4(qb, (q_off + jp * 2048) ^ (uint32_t(ks) << 5));
                mma16816(sacc[2 * jp], ka, qb[0], qb[1]);
                if (2 * jp + 1 < NT) mma16816(sacc[2 * jp + 1 < NT ? 2 * jp + 1 : 0], ka, qb[2], qb[3]);
            }
        }
        // Visibility: keys below p0 are seen by every column; key p0 + r by the columns whose mask has
        // bit r; keys from p0 + T on by none.
        if (key0 + PAGE > p0) {
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t key = key0 + g + 8 * (e >> 1);
                    const uint32_t mask = vmask[j][e & 1];
                    const bool seen = key < p0 || (key < n_keys && ((mask >> (key - p0)) & 1u));
                    if (!seen) sacc[j][e] = -INFINITY;
                }
        }
        // Online softmax with a lazy maximum. A column's running maximum m only has to keep 2^(s - m) in range, not to be
        // the maximum: it is moved (and the sums so far rescaled) only when some score of the page exceeds it by more than
        // 8 -- one vote per page in place of a shuffle reduction per column -- which after a column's first pages is rare.
        // Whatever m a partial ends with, (m, l, o) stay consistent (l = sum 2^(s - m), o = sum 2^(s - m) v), so the merge
        // of warps and of key splits is unchanged. A column's eight lanes (same t) hold the same m: it changes only here,
        // warp-uniformly, from a maximum reduced over those lanes.
        uint32_t pb[NT][2];  // P^T as B operands: b0 keys 2t, 2t + 1; b1 keys 8 + 2t, 9 + 2t; column g of the n-tile
        bool over = false;
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) over = over || fmaxf(sacc[j][e], sacc[j][e + 2]) > m_run[j][e] + 8.0f;
        if (__any_sync(0xffffffffu, over)) {
#pragma unroll
            for (int j = 0; j < NT; j++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    float mx = fmaxf(sacc[j][e], sacc[j][e + 2]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float m_new = fmaxf(m_run[j][e], mx);
                    const float corr = fast_exp2(m_run[j][e] - (m_new == -INFINITY ? 0.0f : m_new));  // 0 for a column's first keys, 1 if nothing moved
                    m_run[j][e] = m_new;
                    l_run[j][e] *= corr;
#pragma unroll
                    for (int dm = 0; dm < 4; dm++) {
                        oacc[dm][j][e] *= corr;
                        oacc[dm][j][e + 2] *= corr;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const float m0 = m_run[j][0] == -INFINITY ? 0.0f : m_run[j][0], m1 = m_run[j][1] == -INFINITY ? 0.0f : m_run[j][1];
            const float p0a = fast_exp2(sacc[j][0] - m0), p0b = fast_exp2(sacc[j][1] - m1);  // key g
            const float p1a = fast_exp2(sacc[j][2] - m0), p1b = fast_exp2(sacc[j][3] - m1);  // key g + 8
            l_run[j][0] += p0a + p1a;
            l_run[j][1] += p0b + p1b;
            pb[j][0] = movmatrix_trans(pack_bf16(p0a, p0b));
            pb[j][1] = movmatrix_trans(pack_bf16(p1a, p1b));
        }
        // O^T += V^T P^T: m-tile dm = dims 16 dm .. 16 dm + 15, one k step of 16 keys.
#pragma unroll
        for (int dm = 0; dm < 4; dm++) {
            uint32_t va[4];
            ldmatrix_x4_trans(va, (vbase + v_off) ^ (uint32_t(dm) << 5));
#pragma unroll
            for (int j = 0; j < NT; j++) mma16816(oacc[dm][j], va, pb[j][0], pb[j][1]);
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
    // its columns to the block's maximum, the block adds them up and writes the partial.
    __syncthreads();
    constexpr int OS = HD + 4;                       // the row stride keeps a quad's stores off each other's banks
    static_assert(size_t(ATTN_WARPS) * NC * (OS + 2) * 4 <= size_t(ATTN_WARPS) * ATTN_STAGES * STAGE_BYTES, "the merge buffers must fit in the stage rings");
    float* ms = reinterpret_cast<float*>(smem);      // [warp][column]
    float* ls = ms + ATTN_WARPS * NC;                // [warp][column], scaled
    float* os = ls + ATTN_WARPS * NC;                // [warp][column][OS], scaled
    if (g == 0) {
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) ms[warp * NC + 8 * j + 2 * t + e] = m_run[j][e];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t col = 8 * j + 2 * t + e;
            float mm = ms[col];
#pragma unroll
            for (int w = 1; w < ATTN_WARPS; w++) mm = fmaxf(mm, ms[w * NC + col]);
            const float wgt = m_run[j][e] == -INFINITY ? 0.0f : fast_exp2(m_run[j][e] - mm);
            float l = l_run[j][e];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            if (g == 0) ls[warp * NC + col] = l * wgt;
#pragma unroll
            for (int dm = 0; dm < 4; dm++) {
                float* o = os + (size_t(warp) * NC + col) * OS + 16 * dm + g;
                o[0] = oacc[dm][j][e] * wgt;
                o[8] = oacc[dm][j][e + 2] * wgt;
            }
        }
    }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < n_cols * HD; idx += blockDim.x) {
        const uint32_t p = idx / HD, d = idx % HD;
        float oo = 0.0f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; w++) oo += os[(size_t(w) * NC + p) * OS + d];
        float* pp = part_of(p);
        if (d == 0) {
            float mm = ms[p], ll = 0.0f;
#pragma unroll
            for (int w = 1; w < ATTN_WARPS; w++) mm = fmaxf(mm, ms[w * NC + p]);
#pragma unroll
            for (int w = 0; w < ATTN_WARPS; w++) ll += ls[w * NC + p];
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
    static PerDevice configured;
    configured.once([smem] {
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        VLT_CUDA(cudaFuncSetAttribute(attn_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    });
    // n8 tiles of query columns the step's longest tile needs (at most VERIFY_T rows x G heads).
    const uint32_t rows = a.max_rows ? std::min(a.max_rows, VERIFY_T) : VERIFY_T, nt = (rows * G + 7) / 8;
    if (nt <= 1) launch_pdl(attn_mma_kernel<1>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
    else if (nt == 2) launch_pdl(attn_mma_kernel<2>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
    else if (nt == 3) launch_pdl(attn_mma_kernel<3>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
    else launch_pdl(attn_mma_kernel<4>, grid, ATTN_WARPS * 32, smem, s, a, *a.maps);
}

}  // namespace vlt
