// The reference architecture's attention on the tensor cores (its `attn_verify`, kernels.metal:891-1167, packs a kv
// head's query heads into the MMA's query dimension the same way, :896).
//
// grid (tokens, kv heads, key splits), four warps. A block takes a contiguous share of the row's keys -- the cached ones
// from its window start (0 on a global layer), then its tile's eight slots under `vis` -- in tiles of 16; warp w takes
// tiles w, w + 4, ... . A tile's K and V rows (16 x 256 bytes each) come into shared memory by per-lane 16-byte
// asynchronous copies (the rows of a ring wrap and a tile need not start on a page boundary, so every row has its own
// address), chunks XOR-swizzled by the row so that ldmatrix meets no bank conflict, in a ring of stages per warp. The
// keys are the MMAs' M side: S^T = K Q^T (16 keys x 8 columns, the columns the G <= 8 query heads of the kv head),
// O^T += V^T P^T (128 dims x 8 columns). q and p enter the MMAs as a bf16 high part plus a bf16 remainder (two MMAs each),
// which keeps 16 bits of them: the reference multiplies in fp32. Online softmax in base 2 with a lazy maximum; the
// partials (m, l, o[128]) per (token, head, split) go to limite::merge_kernel in natural-log units.
#include <algorithm>
#include <cfloat>

#include "kernels.h"
#include "mma.cuh"

namespace vlt {

namespace limite {

constexpr uint32_t D = 128, PART = 132;
constexpr uint32_t TILE = 16, TILE_BYTES = TILE * D * 2, MMA_WARPS = 4, MMA_STAGES = 2;
constexpr uint32_t MMA_SMEM = MMA_WARPS * MMA_STAGES * 2 * TILE_BYTES;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void cluster_sync() { asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of this block's shared-memory location `addr` in block `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// kernels.metal:704-715 `kv_row_of`, in rows of 128 elements.
__device__ __forceinline__ uint32_t kv_row_index(const LimiteKv& kv, uint32_t slot, uint32_t g, uint32_t pos) {
    if (kv.is_global) {
        const uint32_t page = kv.page_table[size_t(slot) * kv.max_pages + (pos >> kv.page_shift)];
        return (((kv.layer * kv.n_pages + page) * kv.n_kv + g) << kv.page_shift) + (pos & ((1u << kv.page_shift) - 1));
    }
    return ((kv.layer * kv.max_seqs + slot) * kv.n_kv + g) * kv.ring + pos % kv.ring;
}

// What a warp carries for one row: Q^T of the kv head's query heads as B operands (column g of the MMA is head g; k step ks
// covers dims 16 ks ..; scaled by scale log2(e), a bf16 high part and a bf16 remainder), and the running softmax of its
// columns 2 tq, 2 tq + 1: O^T [dims 16 dm + g (+ 8)][column], the maximum, and this lane's share of the sum.
struct RowState {
    uint32_t qh[8][2], ql[8][2];
    float oacc[8][4];
    float m_run[2], l_run[2];
};

__device__ __forceinline__ void row_init(RowState& r, const float* __restrict__ q_row, bool valid, float scale_log2, uint32_t tq) {
#pragma unroll
    for (int ks = 0; ks < 8; ks++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float2 v = make_float2(0.0f, 0.0f);
            if (valid) v = *reinterpret_cast<const float2*>(q_row + 16 * ks + 8 * half + 2 * tq);
            v.x *= scale_log2;
            v.y *= scale_log2;
            const uint32_t hi = pack_bf16(v.x, v.y);
            r.qh[ks][half] = hi;
            r.ql[ks][half] = pack_bf16(v.x - bf16lo(hi), v.y - bf16hi(hi));
        }
#pragma unroll
    for (int dm = 0; dm < 8; dm++)
#pragma unroll
        for (int e = 0; e < 4; e++) r.oacc[dm][e] = 0.0f;
    r.m_run[0] = r.m_run[1] = -INFINITY;
    r.l_run[0] = r.l_run[1] = 0.0f;
}

// One tile of 16 keys (K at kbase, V at vbase, rows of 256 bytes, chunks swizzled by the row) against the row: seen0 /
// seen1 say whether the row sees this lane's keys g and g + 8.
// ldmatrix lane roles: matrix lm = lane / 8, row lr = lane % 8. K as A (keys x dims): key 8 (lm & 1) + lr, chunk
// 2 ks + (lm >> 1). V^T as A (dims x keys, .trans): key 8 (lm >> 1) + lr, chunk 2 dm + (lm & 1).
__device__ __forceinline__ void row_tile(RowState& r, uint32_t kbase, uint32_t vbase, bool seen0, bool seen1, uint32_t lane) {
    const uint32_t lm = lane >> 3, lr = lane & 7;
    const uint32_t k_row = (8 * (lm & 1) + lr) * 256, k_c = lm >> 1, v_row = (8 * (lm >> 1) + lr) * 256, v_c = lm & 1;
    float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (uint32_t ks = 0; ks < 8; ks++) {
        uint32_t ka[4];
        ldmatrix_x4(ka, kbase + k_row + (((2 * ks + k_c) ^ lr) << 4));
        mma16816(sacc, ka, r.qh[ks][0], r.qh[ks][1]);
        mma16816(sacc, ka, r.ql[ks][0], r.ql[ks][1]);
    }
    if (!seen0) sacc[0] = sacc[1] = -INFINITY;
    if (!seen1) sacc[2] = sacc[3] = -INFINITY;

    // The running maximum only has to keep 2^(s - m) in range: it moves (and the sums so far are rescaled) only when
    // a score of the tile exceeds it by more than 8, one vote per tile. A column's eight lanes hold the same m.
    bool over = false;
#pragma unroll
    for (int e = 0; e < 2; e++) over = over || fmaxf(sacc[e], sacc[e + 2]) > r.m_run[e] + 8.0f;
    if (__any_sync(0xffffffffu, over)) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            float mx = fmaxf(sacc[e], sacc[e + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(r.m_run[e], mx);
            const float corr = fast_exp2(r.m_run[e] - (m_new == -INFINITY ? 0.0f : m_new));  // 0 for a column's first keys, 1 if nothing moved
            r.m_run[e] = m_new;
            r.l_run[e] *= corr;
#pragma unroll
            for (int dm = 0; dm < 8; dm++) {
                r.oacc[dm][e] *= corr;
                r.oacc[dm][e + 2] *= corr;
            }
        }
    }
    const float m0 = r.m_run[0] == -INFINITY ? 0.0f : r.m_run[0], m1 = r.m_run[1] == -INFINITY ? 0.0f : r.m_run[1];
    const float p0a = fast_exp2(sacc[0] - m0), p0b = fast_exp2(sacc[1] - m1);  // key g
    const float p1a = fast_exp2(sacc[2] - m0), p1b = fast_exp2(sacc[3] - m1);  // key g + 8
    r.l_run[0] += p0a + p1a;
    r.l_run[1] += p0b + p1b;
    // P^T as B operands (b0 keys 2 tq, 2 tq + 1; b1 keys 8 + 2 tq, 9 + 2 tq; column g): high parts and remainders.
    const uint32_t h0 = pack_bf16(p0a, p0b), h1 = pack_bf16(p1a, p1b);
    const uint32_t r0 = pack_bf16(p0a - bf16lo(h0), p0b - bf16hi(h0)), r1 = pack_bf16(p1a - bf16lo(h1), p1b - bf16hi(h1));
    const uint32_t pbh0 = movmatrix_trans(h0), pbh1 = movmatrix_trans(h1), pbl0 = movmatrix_trans(r0), pbl1 = movmatrix_trans(r1);
#pragma unroll
    for (uint32_t dm = 0; dm < 8; dm++) {
        uint32_t va[4];
        ldmatrix_x4_trans(va, vbase + v_row + (((2 * dm + v_c) ^ lr) << 4));
        mma16816(r.oacc[dm], va, pbh0, pbh1);
        mma16816(r.oacc[dm], va, pbl0, pbl1);
    }
}

// The lane's shares of the columns' sums added up over the eight lanes that hold a column.
__device__ __forceinline__ void row_finish(RowState& r) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
        r.l_run[e] += __shfl_xor_sync(0xffffffffu, r.l_run[e], 4);
        r.l_run[e] += __shfl_xor_sync(0xffffffffu, r.l_run[e], 8);
        r.l_run[e] += __shfl_xor_sync(0xffffffffu, r.l_run[e], 16);
    }
}

// One row per block: grid (tokens, kv heads, key splits), four warps that share out the split's tiles. CLUSTER: the
// splits of a (token, kv head) are one thread-block cluster (at most 8 blocks); instead of writing partials for
// merge_kernel, every block stores its heads' (m, l, o) into the first block's shared memory and that block adds them
// up, applies XSA and the gate (kernels.metal:1314-1362 `attn_dec_reduce`) and writes the layer's attention output: no
// second kernel, no round trip of the partials through L2.
template <bool CLUSTER>
__global__ void __launch_bounds__(MMA_WARPS * 32, 3)
    attn_mma_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ vis,
                    const uint16_t* __restrict__ k_cache, const uint16_t* __restrict__ v_cache, const LimiteKv kv, uint32_t n_q, uint32_t window, float scale_log2,
                    uint32_t keys_per_split, uint32_t max_splits, float* part, const float* __restrict__ vdir, const float* __restrict__ gates,
                    const float* __restrict__ xsa, float* out, uint16_t* out_b) {
    pdl_start();
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t t = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z, warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, tq = lane & 3;
    const uint32_t G = n_q / kv.n_kv;
    const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], row = tin[2 * t + 1], mask = vis[t];
    const uint32_t p0 = meta[2 * (t - row % 8) + 1], lo = kv.is_global ? 0u : (pos > window ? pos - window : 0u);  // kernels.metal:809 `key_lo`
    const uint32_t p_run = meta[2 * (t - row) + 1] + (row - row % 8), own = meta[2 * (t - row) + 1] + row;
    const uint32_t n_old = p0 > lo ? p0 - lo : 0, total = n_old + 8;
    const uint32_t begin = sp * keys_per_split, end = min(begin + keys_per_split, total);
    const uint32_t n_tiles = end > begin ? (end - begin + TILE - 1) / TILE : 0;
    const uint32_t my = warp < n_tiles ? (n_tiles - warp + MMA_WARPS - 1) / MMA_WARPS : 0;
    auto seen = [&](uint32_t i) { return i < end && (i < n_old || ((mask >> (i - n_old)) & 1u)); };

    RowState r;
    row_init(r, qkv + size_t(t) * (n_q + 2 * kv.n_kv) * D + size_t(kvh * G + min(g, G - 1)) * D, g < G, scale_log2, tq);

    const uint32_t wbuf = smem_u32(smem) + warp * MMA_STAGES * 2 * TILE_BYTES;
    // Tile i of this warp into stage i % MMA_STAGES. Lanes 0..15 work out the tile's row addresses (an unseen slot or a
    // key past the split reads the row's own key: a valid address, its score masked below); lane l then copies chunk
    // l % 16 of rows 2 j + l / 16.
    auto issue = [&](uint32_t i) {
        const uint32_t i0 = begin + (warp + i * MMA_WARPS) * TILE, idx = i0 + (lane & 15);
        const uint32_t kp = !seen(idx) ? own : idx < n_old ? lo + idx : p_run + (idx - n_old);
        const uint32_t mine = kv_row_index(kv, slot, kvh, kp);
        const uint32_t dst = wbuf + (i % MMA_STAGES) * 2 * TILE_BYTES, chunk = lane & 15;
#pragma unroll
        for (uint32_t j = 0; j < 8; j++) {
            const uint32_t key = 2 * j + (lane >> 4);
            const uint32_t rr = __shfl_sync(0xffffffffu, mine, key);
            const size_t src = size_t(rr) * D + chunk * 8;
            const uint32_t at = dst + key * 256 + ((chunk ^ (key & 7)) << 4);
            cp_async16(at, k_cache + src);
            cp_async16(at + TILE_BYTES, v_cache + src);
        }
    };
    // One group per stage slot, empty ones included, so that "all but the newest MMA_STAGES - 1 groups" is always tile i.
#pragma unroll
    for (uint32_t i = 0; i < MMA_STAGES; i++) {
        if (i < my) issue(i);
        cp_async_commit();
    }
    for (uint32_t i = 0; i < my; i++) {
        cp_async_wait<MMA_STAGES - 1>();
        __syncwarp();
        const uint32_t kbase = wbuf + (i % MMA_STAGES) * 2 * TILE_BYTES;
        const uint32_t i0 = begin + (warp + i * MMA_WARPS) * TILE;
        row_tile(r, kbase, kbase + TILE_BYTES, seen(i0 + g), seen(i0 + g + 8), lane);
        __syncwarp();  // every lane is done with the stage before it is refilled
        if (i + MMA_STAGES < my) issue(i + MMA_STAGES);
        cp_async_commit();
    }
    cp_async_wait<0>();
    row_finish(r);

    // The four warps' sums meet in shared memory (the stage rings are free now); warp w finishes heads w, w + 4, ... .
    __syncthreads();
    constexpr uint32_t OS = D + 4;
    static_assert(MMA_WARPS * 8 * (OS + 2) * 4 <= MMA_SMEM, "the merge buffers must fit in the stage rings");
    float* ms = reinterpret_cast<float*>(smem);  // [warp][column]
    float* ls = ms + MMA_WARPS * 8;              // [warp][column]
    float* os = ls + MMA_WARPS * 8;              // [warp][column][OS]
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const uint32_t col = 2 * tq + e;
        if (col >= G) continue;
        if (g == 0) {
            ms[warp * 8 + col] = r.m_run[e];
            ls[warp * 8 + col] = r.l_run[e];
        }
        float* o = os + (warp * 8 + col) * OS;
#pragma unroll
        for (int dm = 0; dm < 8; dm++) {
            o[16 * dm + g] = r.oacc[dm][e];
            o[16 * dm + g + 8] = r.oacc[dm][e + 2];
        }
    }
    __syncthreads();
    const uint32_t d0 = 4 * lane;
    float mm2[2], ll2[2];  // this warp's heads: warp and warp + MMA_WARPS
    float4 oo2[2];
#pragma unroll
    for (uint32_t hi = 0; hi < 2; hi++) {
        const uint32_t h = warp + hi * MMA_WARPS;
        mm2[hi] = -INFINITY;
        ll2[hi] = 0.0f;
        oo2[hi] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (h >= G) continue;
        float mm = ms[h];
#pragma unroll
        for (uint32_t k = 1; k < MMA_WARPS; k++) mm = fmaxf(mm, ms[k * 8 + h]);
        float ll = 0.0f;
        float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (uint32_t k = 0; k < MMA_WARPS; k++) {
            const float mk = ms[k * 8 + h], wk = mk == -INFINITY ? 0.0f : fast_exp2(mk - mm);
            const float4 ok = *reinterpret_cast<const float4*>(os + (k * 8 + h) * OS + d0);
            ll += ls[k * 8 + h] * wk;
            oo.x += ok.x * wk; oo.y += ok.y * wk; oo.z += ok.z * wk; oo.w += ok.w * wk;
        }
        mm2[hi] = mm;
        ll2[hi] = ll;
        oo2[hi] = oo;
        if (!CLUSTER) {
            float* pp = part + ((size_t(t) * n_q + kvh * G + h) * max_splits + sp) * PART;
            if (lane == 0) { pp[0] = mm * LN2; pp[1] = ll; }  // (-inf stays -inf: an empty split)
            *reinterpret_cast<float4*>(pp + 4 + d0) = oo;
        }
    }
    if (!CLUSTER) return;
    // The cluster's blocks (its ranks are the key splits) meet in the first one's shared memory, [rank][head][PART] over
    // its stage ring: the first barrier says that every block is done with its ring, its own sums read out of it included;
    // the second that every partial is where it will be added up. Every thread of every block reaches both.
    const uint32_t rank = cluster_rank(), n_ranks = gridDim.z;
    static_assert(8 * 8 * PART * 4 <= MMA_SMEM, "the cluster's partials must fit in the stage rings");
    cluster_sync();
#pragma unroll
    for (uint32_t hi = 0; hi < 2; hi++) {
        const uint32_t h = warp + hi * MMA_WARPS;
        if (h >= G) continue;
        const uint32_t dst = cluster_addr(smem_u32(smem) + (rank * 8 + h) * PART * 4, 0);
        if (lane == 0) {
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(mm2[hi]) : "memory");
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + 4), "f"(ll2[hi]) : "memory");
        }
        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (4 + d0) * 4), "f"(oo2[hi].x), "f"(oo2[hi].y), "f"(oo2[hi].z), "f"(oo2[hi].w) : "memory");
    }
    cluster_sync();
    if (rank != 0) return;
    const float* recv = reinterpret_cast<const float*>(smem);
#pragma unroll
    for (uint32_t hi = 0; hi < 2; hi++) {
        const uint32_t h = warp + hi * MMA_WARPS, hq = kvh * G + h;
        if (h >= G) continue;
        float mm = -INFINITY;
        for (uint32_t k = 0; k < n_ranks; k++) mm = fmaxf(mm, recv[(k * 8 + h) * PART]);
        float ll = 0.0f;
        float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t k = 0; k < n_ranks; k++) {
            const float* pk = recv + (k * 8 + h) * PART;
            const float mk = pk[0], wk = mk == -INFINITY ? 0.0f : fast_exp2(mk - mm);
            const float4 ok = *reinterpret_cast<const float4*>(pk + 4 + d0);
            ll += pk[1] * wk;
            oo.x += ok.x * wk; oo.y += ok.y * wk; oo.z += ok.z * wk; oo.w += ok.w * wk;
        }
        oo.x /= ll; oo.y /= ll; oo.z /= ll; oo.w /= ll;
        const float4 vd = *reinterpret_cast<const float4*>(vdir + (size_t(t) * kv.n_kv + kvh) * D + d0);
        const float pr = warp_sum(oo.x * vd.x + oo.y * vd.y + oo.z * vd.z + oo.w * vd.w);
        const float xs = xsa[hq] * pr, gt = gates[size_t(t) * n_q + hq];
        const float4 res = make_float4((oo.x - xs * vd.x) * gt, (oo.y - xs * vd.y) * gt, (oo.z - xs * vd.z) * gt, (oo.w - xs * vd.w) * gt);
        *reinterpret_cast<float4*>(out + (size_t(t) * n_q + hq) * D + d0) = res;
        if (out_b) *reinterpret_cast<uint2*>(out_b + (size_t(t) * n_q + hq) * D + d0) = make_uint2(pack_bf16(res.x, res.y), pack_bf16(res.z, res.w));  // for a tensor-core o projection
    }
}

// A tile of up to eight rows of one run per block -- a verified draft tree or a drafter's block, whose rows share their
// cached keys: grid (tiles, kv heads, key splits), six warps, two blocks an SM. The tile's rows x the kv head's G query
// heads are packed into the MMAs' query dimension (column p = G i + h is row i, head h: kernels.metal:896), at most 48
// columns: warp (grp, kw) takes columns 16 grp .. 16 grp + 15 (two n-tiles) of key tiles kw, kw + 2, ... . The block walks
// the union of its rows' keys (from the smallest window start; then the tile's eight slots) in stages of 32 keys that all
// its threads copy into a ring once, so the cache is read once per tile of rows and a K or V fragment feeds two MMAs;
// Q^T lies in shared memory and comes to the MMAs through ldmatrix. q and p go in as plain bf16 here, as in the plain
// decoder's kernel: with the remainders as well (the one-row kernel's way) the 8 x G columns make this kernel bound by
// mma.sync's rate, 56 us of it for a global layer of 32 streams at 8k against 41 us of memory time. A column's row decides
// what it sees: its own window start and `vis` mask. The key-interleaved warps of a column group meet in shared memory at
// the end. (Two groups of three n-tiles, 242 registers and 8 warps an SM, ran at the same speed.)
constexpr uint32_t ROW_GROUPS = 3, ROW_NT = 2, ROW_CG = 8 * ROW_NT;  // column groups a block's warps split the 48 columns into; n-tiles and columns of one
constexpr uint32_t ROW_KW = 2, ROW_WARPS = ROW_GROUPS * ROW_KW, ROW_STAGES = 4, ROW_COLS = ROW_GROUPS * ROW_CG, ROW_KEYS = ROW_KW * TILE;
constexpr uint32_t ROW_STAGE_BYTES = ROW_KW * 2 * TILE_BYTES;  // a tile per key-interleaved warp, K then V each
constexpr uint32_t ROW_Q_BYTES = (ROW_COLS + 8) * D * 2;  // Q^T; eight rows of padding, which an odd n-tile count's last ldmatrix.x4 would read
constexpr uint32_t ROW_OS = D + 4;
constexpr uint32_t ROW_SMEM = ROW_STAGES * ROW_STAGE_BYTES + ROW_Q_BYTES;
static_assert(ROW_NT <= 4 && ROW_COLS == 48 && ROW_WARPS * 8 * ROW_NT * ROW_OS * 4 <= ROW_SMEM, "the merge buffers must fit in the ring and the Q^T rows");

__global__ void __launch_bounds__(ROW_WARPS * 32, 2)
    attn_mma_rows_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ vis,
                         const uint32_t* __restrict__ tiles, const uint16_t* __restrict__ k_cache, const uint16_t* __restrict__ v_cache, const LimiteKv kv, uint32_t n_q,
                         uint32_t window, float scale_log2, uint32_t keys_per_split, uint32_t max_splits, float* part) {
    pdl_start();
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tile = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z, warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, tq = lane & 3;
    const uint32_t grp = warp % ROW_GROUPS, kw = warp / ROW_GROUPS;
    const uint32_t G = n_q / kv.n_kv;
    const uint32_t t0 = tiles[2 * tile], T = tiles[2 * tile + 1], n_cols = T * G;
    const uint32_t slot = meta[2 * t0], row0 = tin[2 * t0 + 1];
    const uint32_t p0 = meta[2 * t0 + 1], p_run = meta[2 * (t0 - row0) + 1] + row0;  // the tile's first position; its first row's place in the cache
    auto lo_of = [&](uint32_t p) { return kv.is_global ? 0u : (p > window ? p - window : 0u); };  // kernels.metal:809 `key_lo`
    uint32_t lo_min = lo_of(p0), lo_max = lo_min;
    for (uint32_t i = 1; i < T; i++) {
        const uint32_t l = lo_of(meta[2 * (t0 + i) + 1]);
        lo_min = min(lo_min, l);
        lo_max = max(lo_max, l);
    }
    const uint32_t n_old = p0 > lo_min ? p0 - lo_min : 0, total = n_old + 8;
    const uint32_t begin = sp * keys_per_split, end = min(begin + keys_per_split, total);
    const uint32_t n_stages = end > begin ? (end - begin + ROW_KEYS - 1) / ROW_KEYS : 0;

    // Q^T into shared memory as [column][128 dims] bf16, 16-byte chunks swizzled by the row.
    const uint32_t ring = smem_u32(smem), q_hi = ring + ROW_STAGES * ROW_STAGE_BYTES;
    for (uint32_t c = threadIdx.x; c < ROW_COLS * 16; c += ROW_WARPS * 32) {
        const uint32_t pcol = c / 16, chunk = c % 16;
        uint4 hi = make_uint4(0, 0, 0, 0);
        if (pcol < n_cols) {
            const float* qp = qkv + size_t(t0 + pcol / G) * (n_q + 2 * kv.n_kv) * D + size_t(kvh * G + pcol % G) * D + chunk * 8;
            const float4 a = *reinterpret_cast<const float4*>(qp), bq = *reinterpret_cast<const float4*>(qp + 4);
            const float v[8] = {a.x * scale_log2, a.y * scale_log2, a.z * scale_log2, a.w * scale_log2, bq.x * scale_log2, bq.y * scale_log2, bq.z * scale_log2, bq.w * scale_log2};
            hi = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
        const uint32_t off = pcol * 256 + ((chunk ^ (pcol & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + ROW_STAGES * ROW_STAGE_BYTES + off) = hi;
    }

    // This lane's columns: ROW_CG grp + 8 j + 2 tq (+ 1) of n-tile j; the window start and the mask of each one's row.
    uint32_t c_lo[ROW_NT][2], c_mask[ROW_NT][2];
#pragma unroll
    for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t pcol = ROW_CG * grp + 8 * j + 2 * tq + e;
            const bool real = pcol < n_cols;
            const uint32_t t = t0 + (real ? pcol / G : 0);
            c_lo[j][e] = real ? lo_of(meta[2 * t + 1]) : 0xffffffffu;  // (a column that is none sees nothing)
            c_mask[j][e] = real ? vis[t] : 0u;
        }

    // Stage i: keys begin + ROW_KEYS i ..; thread j copies chunk j % 16 of keys j / 16 + 8 u, K and V (a key past the split, or a
    // slot past the tile's rows, which has no place in the cache, reads the tile's first row's own key: a valid address
    // that no column sees).
    auto issue = [&](uint32_t i) {
        const uint32_t chunk = threadIdx.x & 15, first = begin + i * ROW_KEYS, p_first = lo_min + first;
        // A stage of cached keys that lie in one page, or in one stretch of the ring, takes one address and counts on.
        const bool together = first + ROW_KEYS <= n_old && first + ROW_KEYS <= end &&
                              (kv.is_global ? (p_first >> kv.page_shift) == ((p_first + ROW_KEYS - 1) >> kv.page_shift) : p_first % kv.ring + ROW_KEYS <= kv.ring);
        const uint32_t row_first = together ? kv_row_index(kv, slot, kvh, p_first) : 0u;
#pragma unroll
        for (uint32_t u = 0; u < (ROW_KEYS + ROW_WARPS * 2 - 1) / (ROW_WARPS * 2); u++) {
            const uint32_t key = (threadIdx.x >> 4) + ROW_WARPS * 2 * u, idx = first + key;
            if (key >= ROW_KEYS) break;
            uint32_t rowi = row_first + key;
            if (!together) {
                const uint32_t kp = idx >= end ? p_run : idx < n_old ? lo_min + idx : p_run + (idx - n_old < T ? idx - n_old : 0u);
                rowi = kv_row_index(kv, slot, kvh, kp);
            }
            const size_t src = size_t(rowi) * D + chunk * 8;
            const uint32_t at = ring + (i % ROW_STAGES) * ROW_STAGE_BYTES + (key >> 4) * 2 * TILE_BYTES + (key & 15) * 256 + ((chunk ^ (key & 7)) << 4);
            cp_async16(at, k_cache + src);
            cp_async16(at + TILE_BYTES, v_cache + src);
        }
    };
    // One group per iteration, empty ones included: at iteration i all but the newest ROW_STAGES - 2 groups are complete,
    // which is stage i; the barrier that follows also says that every warp is done with stage i - 1, which the new copy takes.
#pragma unroll
    for (uint32_t i = 0; i + 1 < ROW_STAGES; i++) {
        if (i < n_stages) issue(i);
        cp_async_commit();
    }

    const uint32_t lm = lane >> 3, lr = lane & 7;
    const uint32_t k_row = (8 * (lm & 1) + lr) * 256, k_c = lm >> 1, v_row = (8 * (lm >> 1) + lr) * 256, v_c = lm & 1;
    // Q^T as B: one ldmatrix.x4 brings b0, b1 of n-tile jq and of jq + 1: matrix lm -> column ROW_CG grp + 8 (jq + (lm >> 1)) + lr,
    // chunk 2 ks + (lm & 1).
    const uint32_t q_row = (ROW_CG * grp + 8 * (lm >> 1) + lr) * 256, q_c = lm & 1;

    float oacc[8][ROW_NT][4];
    float m_run[ROW_NT][2], l_run[ROW_NT][2];
#pragma unroll
    for (int j = 0; j < int(ROW_NT); j++) {
#pragma unroll
        for (int dm = 0; dm < 8; dm++)
#pragma unroll
            for (int e = 0; e < 4; e++) oacc[dm][j][e] = 0.0f;
        m_run[j][0] = m_run[j][1] = -INFINITY;
        l_run[j][0] = l_run[j][1] = 0.0f;
    }

    for (uint32_t i = 0; i < n_stages; i++) {
        cp_async_wait<ROW_STAGES - 2>();
        __syncthreads();  // (the first one also covers the Q^T stores)
        const uint32_t i0 = begin + i * ROW_KEYS + kw * TILE;  // this warp's tile of the stage
        if (i0 >= end) {
            if (i + ROW_STAGES - 1 < n_stages) issue(i + ROW_STAGES - 1);
            cp_async_commit();
            continue;
        }
        const uint32_t kbase = ring + (i % ROW_STAGES) * ROW_STAGE_BYTES + kw * 2 * TILE_BYTES, vbase = kbase + TILE_BYTES;

        float sacc[ROW_NT][4];
#pragma unroll
        for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
            for (int e = 0; e < 4; e++) sacc[j][e] = 0.0f;
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ks++) {
            uint32_t ka[4];
            ldmatrix_x4(ka, kbase + k_row + (((2 * ks + k_c) ^ lr) << 4));
            const uint32_t qoff = q_row + (((2 * ks + q_c) ^ lr) << 4);
#pragma unroll
            for (uint32_t jq = 0; jq < ROW_NT; jq += 2) {  // (an odd count's last load also reads the eight rows after its n-tile: unused)
                uint32_t qa[4];
                ldmatrix_x4(qa, q_hi + qoff + jq * 8 * 256);
                mma16816(sacc[jq], ka, qa[0], qa[1]);
                if (jq + 1 < ROW_NT) mma16816(sacc[jq + 1 < ROW_NT ? jq + 1 : jq], ka, qa[2], qa[3]);
            }
        }
        // Who sees what: nothing to do for a tile of cached keys inside every row's window.
        if (i0 + TILE > n_old || i0 + TILE > end || lo_min + i0 < lo_max) {
#pragma unroll
            for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t idx = i0 + g + 8 * (e >> 1);
                    const bool seen = idx < end && (idx < n_old ? lo_min + idx >= c_lo[j][e & 1] : ((c_mask[j][e & 1] >> (idx - n_old)) & 1u) != 0);
                    if (!seen) sacc[j][e] = -INFINITY;
                }
        } else {
#pragma unroll
            for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (c_lo[j][e & 1] == 0xffffffffu) sacc[j][e] = -INFINITY;  // (no such column)
        }
        bool over = false;
#pragma unroll
        for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
            for (int e = 0; e < 2; e++) over = over || fmaxf(sacc[j][e], sacc[j][e + 2]) > m_run[j][e] + 8.0f;
        if (__any_sync(0xffffffffu, over)) {
#pragma unroll
            for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    float mx = fmaxf(sacc[j][e], sacc[j][e + 2]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float m_new = fmaxf(m_run[j][e], mx);
                    const float corr = fast_exp2(m_run[j][e] - (m_new == -INFINITY ? 0.0f : m_new));
                    m_run[j][e] = m_new;
                    l_run[j][e] *= corr;
#pragma unroll
                    for (int dm = 0; dm < 8; dm++) {
                        oacc[dm][j][e] *= corr;
                        oacc[dm][j][e + 2] *= corr;
                    }
                }
        }
        uint32_t pbh[ROW_NT][2];
#pragma unroll
        for (int j = 0; j < int(ROW_NT); j++) {
            const float m0 = m_run[j][0] == -INFINITY ? 0.0f : m_run[j][0], m1 = m_run[j][1] == -INFINITY ? 0.0f : m_run[j][1];
            const float p0a = fast_exp2(sacc[j][0] - m0), p0b = fast_exp2(sacc[j][1] - m1);  // key g
            const float p1a = fast_exp2(sacc[j][2] - m0), p1b = fast_exp2(sacc[j][3] - m1);  // key g + 8
            l_run[j][0] += p0a + p1a;
            l_run[j][1] += p0b + p1b;
            pbh[j][0] = movmatrix_trans(pack_bf16(p0a, p0b));
            pbh[j][1] = movmatrix_trans(pack_bf16(p1a, p1b));
        }
#pragma unroll
        for (uint32_t dm = 0; dm < 8; dm++) {
            uint32_t va[4];
            ldmatrix_x4_trans(va, vbase + v_row + (((2 * dm + v_c) ^ lr) << 4));
#pragma unroll
            for (int j = 0; j < int(ROW_NT); j++) mma16816(oacc[dm][j], va, pbh[j][0], pbh[j][1]);
        }
        // The next copies go out behind the arithmetic (their addresses take a page-table load each), into the stage every
        // warp left before this iteration's barrier.
        if (i + ROW_STAGES - 1 < n_stages) issue(i + ROW_STAGES - 1);
        cp_async_commit();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            l_run[j][e] += __shfl_xor_sync(0xffffffffu, l_run[j][e], 4);
            l_run[j][e] += __shfl_xor_sync(0xffffffffu, l_run[j][e], 8);
            l_run[j][e] += __shfl_xor_sync(0xffffffffu, l_run[j][e], 16);
        }
    __syncthreads();  // the ring and the Q^T copies are free: every warp lays its columns' partials out in them
    float* os = reinterpret_cast<float*>(smem);  // [warp][ROW_CG columns][ROW_OS]: o[128], then m and l
#pragma unroll
    for (int j = 0; j < int(ROW_NT); j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t lc = 8 * j + 2 * tq + e;
            if (ROW_CG * grp + lc >= n_cols) continue;
            float* o = os + (warp * ROW_CG + lc) * ROW_OS;
            if (g == 0) {
                o[D] = m_run[j][e];
                o[D + 1] = l_run[j][e];
            }
#pragma unroll
            for (int dm = 0; dm < 8; dm++) {
                o[16 * dm + g] = oacc[dm][j][e];
                o[16 * dm + g + 8] = oacc[dm][j][e + 2];
            }
        }
    __syncthreads();
    // The key-interleaved warps of a column group added up per column: warp w takes columns w, w + ROW_WARPS, ... of the tile.
    const uint32_t d0 = 4 * lane;
    for (uint32_t pcol = warp; pcol < n_cols; pcol += ROW_WARPS) {
        const uint32_t cg = pcol / ROW_CG, lc = pcol % ROW_CG;
        float mm = -INFINITY;
#pragma unroll
        for (uint32_t k = 0; k < ROW_KW; k++) mm = fmaxf(mm, os[((ROW_GROUPS * k + cg) * ROW_CG + lc) * ROW_OS + D]);
        float ll = 0.0f;
        float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (uint32_t k = 0; k < ROW_KW; k++) {
            const float* o = os + ((ROW_GROUPS * k + cg) * ROW_CG + lc) * ROW_OS;
            const float mk = o[D], wk = mk == -INFINITY ? 0.0f : fast_exp2(mk - mm);
            const float4 ok = *reinterpret_cast<const float4*>(o + d0);
            ll += o[D + 1] * wk;
            oo.x += ok.x * wk; oo.y += ok.y * wk; oo.z += ok.z * wk; oo.w += ok.w * wk;
        }
        float* pp = part + ((size_t(t0 + pcol / G) * n_q + kvh * G + pcol % G) * max_splits + sp) * PART;
        if (lane == 0) { pp[0] = mm * LN2; pp[1] = ll; }  // (-inf stays -inf: nothing seen in this split)
        *reinterpret_cast<float4*>(pp + 4 + d0) = oo;
    }
}

}  // namespace limite

// The launches: keys_per_split a multiple of 64 (a tile per warp and round) for the one-row kernel, of 16 for the rows' one.
void launch_limite_attn_mma(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint16_t* k_cache, const uint16_t* v_cache,
                            const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, uint32_t n, uint32_t keys_per_split, uint32_t splits, float* part,
                            cudaStream_t s) {
    static PerDevice configured;
    configured.once([] { VLT_CUDA(cudaFuncSetAttribute(limite::attn_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(limite::MMA_SMEM))); });
    launch_pdl(limite::attn_mma_kernel<false>, dim3(n, kv.n_kv, splits), limite::MMA_WARPS * 32, limite::MMA_SMEM, s, qkv, meta, tin, vis, k_cache, v_cache, kv, n_q,
               window, scale * limite::LOG2E, keys_per_split, splits, part, static_cast<const float*>(nullptr), static_cast<const float*>(nullptr),
               static_cast<const float*>(nullptr), static_cast<float*>(nullptr), static_cast<uint16_t*>(nullptr));
}
// The same with a (token, kv head)'s splits (at most 8) as a thread-block cluster that finishes the attention itself.
void launch_limite_attn_cluster(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint16_t* k_cache, const uint16_t* v_cache,
                                const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, const float* vdir, const float* gates, const float* xsa, uint32_t n,
                                uint32_t keys_per_split, uint32_t splits, float* out, uint16_t* out_b, cudaStream_t s) {
    if (splits < 1 || splits > 8) throw Error("internal: a cluster of 1..8 key splits");
    static PerDevice configured;
    configured.once([] { VLT_CUDA(cudaFuncSetAttribute(limite::attn_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(limite::MMA_SMEM))); });
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n, kv.n_kv, splits);
    cfg.blockDim = dim3(limite::MMA_WARPS * 32);
    cfg.dynamicSmemBytes = limite::MMA_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = splits;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    VLT_CUDA(cudaLaunchKernelEx(&cfg, limite::attn_mma_kernel<true>, qkv, meta, tin, vis, k_cache, v_cache, kv, n_q, window, scale * limite::LOG2E, keys_per_split, splits,
                                static_cast<float*>(nullptr), vdir, gates, xsa, out, out_b));
    launch_counter().fetch_add(1, std::memory_order_relaxed);
}
void launch_limite_attn_rows(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint32_t* tiles, const uint16_t* k_cache,
                             const uint16_t* v_cache, const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, uint32_t n_tiles, uint32_t keys_per_split,
                             uint32_t splits, float* part, cudaStream_t s) {
    static PerDevice configured;
    configured.once([] { VLT_CUDA(cudaFuncSetAttribute(limite::attn_mma_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(limite::ROW_SMEM))); });
    launch_pdl(limite::attn_mma_rows_kernel, dim3(n_tiles, kv.n_kv, splits), limite::ROW_WARPS * 32, limite::ROW_SMEM, s, qkv, meta, tin, vis, tiles, k_cache, v_cache, kv,
               n_q, window, scale * limite::LOG2E, keys_per_split, splits, part);
}

}  // namespace vlt
