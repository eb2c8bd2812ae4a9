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

// One row per block: grid (tokens, kv heads, key splits), four warps that share out the split's tiles.
__global__ void __launch_bounds__(MMA_WARPS * 32, 3)
    attn_mma_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ vis,
                    const uint16_t* __restrict__ k_cache, const uint16_t* __restrict__ v_cache, const LimiteKv kv, uint32_t n_q, uint32_t window, float scale_log2,
                    uint32_t keys_per_split, uint32_t max_splits, float* part) {
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
    for (uint32_t h = warp; h < G; h += MMA_WARPS) {
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
        float* pp = part + ((size_t(t) * n_q + kvh * G + h) * max_splits + sp) * PART;
        if (lane == 0) { pp[0] = mm * LN2; pp[1] = ll; }  // (-inf stays -inf: an empty split)
        *reinterpret_cast<float4*>(pp + 4 + d0) = oo;
    }
}

// A tile of up to eight rows of one run per block -- a verified draft tree, whose rows share their cached keys: grid
// (tiles, kv heads, key splits), eight warps, warp w the tile's row w. The block walks the union of its rows' keys (from
// the smallest window start; then the tile's eight slots) in tiles of 16 that all 256 threads copy into a ring of stages
// once, and every warp multiplies each tile with its own row under that row's window start and `vis` mask, so the cache
// is read once per tile of rows and not once per row. No meeting of warps at the end: a warp holds its row's whole
// partial for the split.
constexpr uint32_t ROW_WARPS = 8, ROW_STAGES = 4;
constexpr uint32_t ROW_OS = D + 4;
constexpr uint32_t ROW_SMEM = ROW_STAGES * 2 * TILE_BYTES > ROW_WARPS * 8 * ROW_OS * 4 ? ROW_STAGES * 2 * TILE_BYTES : ROW_WARPS * 8 * ROW_OS * 4;

__global__ void __launch_bounds__(ROW_WARPS * 32, 1)
    attn_mma_rows_kernel(const float* __restrict__ qkv, const uint32_t* __restrict__ meta, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ vis,
                         const uint32_t* __restrict__ tiles, const uint16_t* __restrict__ k_cache, const uint16_t* __restrict__ v_cache, const LimiteKv kv, uint32_t n_q,
                         uint32_t window, float scale_log2, uint32_t keys_per_split, uint32_t max_splits, float* part) {
    pdl_start();
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tile = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z, warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, tq = lane & 3;
    const uint32_t G = n_q / kv.n_kv;
    const uint32_t t0 = tiles[2 * tile], T = tiles[2 * tile + 1];
    const bool has_row = warp < T;
    const uint32_t t = t0 + (has_row ? warp : 0);  // (a warp without a row walks along with row 0's numbers and writes nothing)
    const uint32_t slot = meta[2 * t0], row0 = tin[2 * t0 + 1];
    const uint32_t p0 = meta[2 * t0 + 1], p_run = meta[2 * (t0 - row0) + 1] + row0;  // the tile's first position; its first row's place in the cache
    const uint32_t pos = meta[2 * t + 1], mask = has_row ? vis[t] : 0u;
    auto lo_of = [&](uint32_t p) { return kv.is_global ? 0u : (p > window ? p - window : 0u); };  // kernels.metal:809 `key_lo`
    const uint32_t lo = lo_of(pos);
    uint32_t lo_min = lo_of(p0);
    for (uint32_t i = 1; i < T; i++) lo_min = min(lo_min, lo_of(meta[2 * (t0 + i) + 1]));
    const uint32_t n_old = p0 > lo_min ? p0 - lo_min : 0, total = n_old + 8;
    const uint32_t begin = sp * keys_per_split, end = min(begin + keys_per_split, total);
    const uint32_t n_tiles = end > begin ? (end - begin + TILE - 1) / TILE : 0;
    // Key i of the block's walk: cached position lo_min + i below n_old, then the tile's slot i - n_old.
    auto in_walk = [&](uint32_t i) { return i < end; };
    auto seen = [&](uint32_t i) { return has_row && i < end && (i < n_old ? lo_min + i >= lo : ((mask >> (i - n_old)) & 1u) != 0); };

    RowState r;
    row_init(r, qkv + size_t(t) * (n_q + 2 * kv.n_kv) * D + size_t(kvh * G + min(g, G - 1)) * D, has_row && g < G, scale_log2, tq);

    const uint32_t ring = smem_u32(smem);
    // Tile i into stage i % ROW_STAGES: thread j copies chunk j % 16 of key j / 16, K and V (a key past the split reads
    // the tile's first row's own key: a valid address, masked for every row).
    auto issue = [&](uint32_t i) {
        const uint32_t key = threadIdx.x >> 4, chunk = threadIdx.x & 15, idx = begin + i * TILE + key;
        // (a slot past the tile's rows has no place in the cache: it reads the first row's, and no row's mask names it)
        const uint32_t kp = !in_walk(idx) ? p_run : idx < n_old ? lo_min + idx : p_run + (idx - n_old < T ? idx - n_old : 0u);
        const size_t src = size_t(kv_row_index(kv, slot, kvh, kp)) * D + chunk * 8;
        const uint32_t at = ring + (i % ROW_STAGES) * 2 * TILE_BYTES + key * 256 + ((chunk ^ (key & 7)) << 4);
        cp_async16(at, k_cache + src);
        cp_async16(at + TILE_BYTES, v_cache + src);
    };
    // One group per iteration, empty ones included: at iteration i all but the newest ROW_STAGES - 2 groups are complete,
    // which is tile i; the barrier that follows also says that every warp is done with tile i - 1, whose stage the new
    // copy takes.
#pragma unroll
    for (uint32_t i = 0; i + 1 < ROW_STAGES; i++) {
        if (i < n_tiles) issue(i);
        cp_async_commit();
    }
    for (uint32_t i = 0; i < n_tiles; i++) {
        cp_async_wait<ROW_STAGES - 2>();
        __syncthreads();
        if (i + ROW_STAGES - 1 < n_tiles) issue(i + ROW_STAGES - 1);
        cp_async_commit();
        if (!has_row) continue;
        const uint32_t kbase = ring + (i % ROW_STAGES) * 2 * TILE_BYTES, i0 = begin + i * TILE;
        row_tile(r, kbase, kbase + TILE_BYTES, seen(i0 + g), seen(i0 + g + 8), lane);
    }
    cp_async_wait<0>();
    row_finish(r);
    __syncthreads();  // the ring is free: each warp lays its row's partial out in it, then writes it in whole rows
    if (!has_row) return;
    float* os = reinterpret_cast<float*>(smem) + warp * 8 * ROW_OS;  // [column][ROW_OS]: o[128], then m and l
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const uint32_t col = 2 * tq + e;
        if (col >= G) continue;
        float* o = os + col * ROW_OS;
        if (g == 0) {
            o[D] = r.m_run[e];
            o[D + 1] = r.l_run[e];
        }
#pragma unroll
        for (int dm = 0; dm < 8; dm++) {
            o[16 * dm + g] = r.oacc[dm][e];
            o[16 * dm + g + 8] = r.oacc[dm][e + 2];
        }
    }
    __syncwarp();
    const uint32_t d0 = 4 * lane;
    for (uint32_t h = 0; h < G; h++) {
        const float* o = os + h * ROW_OS;
        float* pp = part + ((size_t(t) * n_q + kvh * G + h) * max_splits + sp) * PART;
        if (lane == 0) { pp[0] = o[D] * LN2; pp[1] = o[D + 1]; }  // (-inf stays -inf: nothing seen in this split)
        *reinterpret_cast<float4*>(pp + 4 + d0) = *reinterpret_cast<const float4*>(o + d0);
    }
}

}  // namespace limite

// The launches: keys_per_split a multiple of 64 (a tile per warp and round) for the one-row kernel, of 16 for the rows' one.
void launch_limite_attn_mma(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint16_t* k_cache, const uint16_t* v_cache,
                            const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, uint32_t n, uint32_t keys_per_split, uint32_t splits, float* part,
                            cudaStream_t s) {
    static PerDevice configured;
    configured.once([] { VLT_CUDA(cudaFuncSetAttribute(limite::attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(limite::MMA_SMEM))); });
    launch_pdl(limite::attn_mma_kernel, dim3(n, kv.n_kv, splits), limite::MMA_WARPS * 32, limite::MMA_SMEM, s, qkv, meta, tin, vis, k_cache, v_cache, kv, n_q, window,
               scale * limite::LOG2E, keys_per_split, splits, part);
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
