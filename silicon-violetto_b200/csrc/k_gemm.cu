// The verify GEMM on the 5th-generation tensor cores: Y[t][row] = epilogue(W[row] . Xb[t]) for
// steps of 16 to 256 tokens (S streams x k+1 rows). The reference's tiled GEMM
// (kernels.metal:319-514) stages k tiles through threadgroup memory and dequantises on the way;
// here
//   - the weight tile is the MMA's M side (128 rows) and the tokens its N side (16..256), so a
//     weight is read from HBM once whatever the number of streams;
//   - operands come in by TMA (no multicast) into 128-byte-swizzled shared memory, a ring of
//     stages guarded by mbarriers; tcgen05.mma, issued by one thread, accumulates fp32 in TMEM;
//   - int8 weights arrive as raw bytes in a ring of their own; sixteen warps, in four groups that
//     take k blocks in turn, turn each into bf16 (exactly) and store it into tensor memory, where
//     the MMA takes its A operand from; the scale per output row is applied in the epilogue;
//   - the epilogue warps read TMEM with tcgen05.ld and apply the fused epilogues (RMSNorm scale,
//     residual add, SwiGLU on interleaved gate/up rows, head) before the coalesced store.
// Every wait is bounded: on a time-out the kernel sets the error flag, frees its TMEM and returns.
#include <cuda.h>

#include <algorithm>
#include <map>
#include <tuple>

#include "kernels.h"

namespace vlt {

namespace gemm {

constexpr uint32_t BM = 128, BK = 64;
constexpr uint32_t CONV_WPG = 4;  // converter warps per group: one per quarter of the TMEM lanes
constexpr uint32_t FIRST_CONV = 3;
// warp 0: weight TMA, warp 1: MMA, warp 2: activation TMA, the rest (CW of them, in groups that each take their own k
// block): conversion and epilogue. Sixteen normally, one block per SM. Eight -- two blocks per SM, each with half the
// shared and tensor memory -- for a GEMM of several waves of tiles (the head over the vocabulary): one block's fill and
// epilogue then run under the other's main loop.
constexpr uint32_t threads_of(uint32_t cw) { return 32 * (FIRST_CONV + cw); }
constexpr uint32_t SPIN = 1u << 26;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x),
                 "r"(y), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 64 bf16; groups of
// 8 rows are 1024 bytes apart. Bits: [0,14) address >> 4, [16,30) leading offset >> 4 (unused for
// swizzled K-major), [32,46) stride offset >> 4, [46,48) version 1, [61,64) swizzle mode 2 (128 B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor for kind::f16: fp32 accumulate, bf16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d), "l"(adesc), "l"(bdesc),
                 "r"(idesc), "r"(accumulate)
                 : "memory");
}
// The same with A in tensor memory: lane = row, a 32-bit column = two consecutive k.
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc),
                 "r"(idesc), "r"(accumulate)
                 : "memory");
}
// 32 columns of this warp's 32 lanes from registers (thread = lane, register j = column j).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
        "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// One lane of a converged warp (the same one every time).
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}" : "=r"(pred));
    return pred;
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// Four int8 (one word) to two bf16 pairs, exactly (see k_matmul.cu).
__device__ __forceinline__ void cvt_i8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
    lo = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
    hi = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

struct Maps {
    alignas(64) uint8_t a[128];
    alignas(64) uint8_t b[128];
};

struct Args {
    MatArgs m;
    uint32_t n_pad;     // tokens rounded up to 16: the MMA's N
    uint32_t stages_a;    // A stages: in shared memory (bf16 weights) or in tensor memory (int8 weights)
    uint32_t stages_b;    // B stages in shared memory
    uint32_t raw_stages;  // int8 only: raw weight stages in front of the A stages
    uint32_t tmem_cols; // power of two >= 32 holding the accumulator and, for int8, the A stages
    uint32_t tmem_a0;   // int8: the first A stage's column (32 columns per stage)
    uint32_t splits;    // blocks of a cluster that share a weight tile, each over a slice of k
    uint32_t* err_flag;
};

}  // namespace gemm


namespace gemm {

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    for (uint32_t i = 0; i < SPIN; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
#ifdef VLT_GEMM_PROBE
__device__ unsigned long long g_probe[8][64];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define PROBE(e, i) do { if (blockIdx.x == 0 && (i) < 64) g_probe[e][i] = gtime(); } while (0)
#else
#define PROBE(e, i) do { } while (0)
#endif
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of this block's shared-memory location `addr` in block `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster(uint32_t addr) {
    float v;
    asm("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));  // ordered by the cluster barrier before it
    return v;
}

// grid: (m / 128) * splits blocks in clusters of `splits`. A cluster owns a 128-row weight tile;
// its blocks each stream a slice of k into their own TMEM accumulator, send every group of 16 tokens
// to the block that finishes it (stores into its shared memory), and each then adds up, in rank
// order, the groups it owns.
template <bool INT8, uint32_t EPI, uint32_t CONV_WARPS = 16>
__global__ void __launch_bounds__(threads_of(CONV_WARPS), CONV_WARPS == 16 ? 1 : 2) gemm_kernel(const __grid_constant__ Maps maps, const Args a) {
    constexpr uint32_t CONV_GROUPS = CONV_WARPS / CONV_WPG;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Three rings, each as deep as its own latency asks. B stages (n_pad x 128 B) in shared memory cover
    // an L2 round trip. A stages: bf16 weights land in shared memory (16 KiB a stage); int8 weights are
    // converted into tensor memory (32 columns a stage, behind the accumulator), so shared memory carries
    // a weight byte once, not five times. In front of those, int8 weights have `R` raw stages of 8 KiB:
    // the bytes in flight that cover the latency of HBM.
    const uint32_t n_pad = a.n_pad, CA = a.stages_a, CB = a.stages_b, R = INT8 ? a.raw_stages : 0, splits = a.splits;
    const uint32_t a_bytes = BM * BK * 2, b_bytes = n_pad * BK * 2, raw_bytes = BM * BK;
    const uint32_t a_region = INT8 ? 0 : CA * a_bytes;
    // The split-k exchange buffer reuses the rings: [splits][groups of 16 tokens a block finishes][16][128] floats.
    const uint32_t ring_bytes = max(a_region + CB * b_bytes + R * raw_bytes, splits * ((n_pad / 16) / splits + 1) * 16 * BM * 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ring_bytes);
    // a_full[CA], a_empty[CA], b_full[CB], b_empty[CB], raw_full[R], raw_empty[R], then the accumulator's barrier
    const uint32_t bar_afull = smem_u32(bars), bar_aempty = bar_afull + 8 * CA, bar_bfull = bar_aempty + 8 * CA, bar_bempty = bar_bfull + 8 * CB,
                   bar_rfull = bar_bempty + 8 * CB, bar_rempty = bar_rfull + 8 * R, bar_accum = bar_rempty + 8 * R;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * CA + 2 * CB + 2 * R + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* inv_s = reinterpret_cast<float*>(const_cast<uint32_t*>(tmem_slot) + 2);  // 1/rms per token
    uint32_t* pos_s = reinterpret_cast<uint32_t*>(inv_s + n_pad);                    // EPI_QKV: the token's position ...
    uint32_t* kvrow_s = pos_s + n_pad;  // ... and the cache row (of 64 elements) of its kv head 0, NO_TOK if it writes none
    float* ssq_s = reinterpret_cast<float*>(kvrow_s + n_pad);  // EPI_RESID with ssq_out: [row group of 32][token] sums of y^2
    const uint32_t smem_base = smem_u32(smem);
    auto stage_a = [&](uint32_t c) { return smem_base + c * a_bytes; };
    auto stage_b = [&](uint32_t c) { return smem_base + a_region + c * b_bytes; };
    auto stage_raw = [&](uint32_t r) { return smem_base + a_region + CB * b_bytes + r * raw_bytes; };

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t rank = splits > 1 ? cluster_rank() : 0, tile = blockIdx.x / splits;
    const uint32_t row0 = tile * BM, nkb_all = a.m.k / BK;
    // This block's k blocks: an even share, the first ranks one more.
    const uint32_t kb_begin = rank * (nkb_all / splits) + min(rank, nkb_all % splits);
    const uint32_t nkb = nkb_all / splits + (rank < nkb_all % splits ? 1 : 0);

    if (tid == 0) {
        for (uint32_t c = 0; c < CA; c++) {
            mbar_init(bar_afull + 8 * c, INT8 ? CONV_WPG : 1);  // a group's converter warps, or the loader's expect_tx
            mbar_init(bar_aempty + 8 * c, 1);
        }
        for (uint32_t c = 0; c < CB; c++) {
            mbar_init(bar_bfull + 8 * c, 1);
            mbar_init(bar_bempty + 8 * c, 1);
        }
        for (uint32_t r = 0; r < R; r++) {
            mbar_init(bar_rfull + 8 * r, 1);
            mbar_init(bar_rempty + 8 * r, CONV_WPG);
        }
        mbar_init(bar_accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    // Programmatic dependent launch: the kernel queued behind this one may start its own set-up and weight
    // loads now; and this one, if it was started that way, has touched nothing yet that the kernel before it
    // writes -- the weights' loader, the converters and the MMA issuer never do, the activations' loader and
    // the epilogue warps wait for that kernel first (griddepcontrol.wait).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // The loops below keep their stage index and phase bit by increment: a thread that feeds the tensor
    // core runs alone in its warp, and every division or descriptor rebuilt per k block is on the critical path.
    if (warp == 0) {
        // The weights' loader: raw int8 tiles into the deep ring, or bf16 tiles straight into the operand ring.
        if (lane == 0) {
            const uint32_t n_st = INT8 ? R : CA, bar_e = INT8 ? bar_rempty : bar_aempty, bar_f = INT8 ? bar_rfull : bar_afull;
            const uint32_t dst0 = INT8 ? stage_raw(0) : stage_a(0), step = INT8 ? raw_bytes : a_bytes, bytes = step;
            uint32_t st = 0, ph = 1;
            for (uint32_t i = 0; i < nkb; i++) {
                ok = wait_or_abort(bar_e + 8 * st, ph, abort_flag);
                if (!ok) break;
                PROBE(0, i);
                mbar_expect_tx(bar_f + 8 * st, bytes);
                tma_load_2d(dst0 + st * step, &maps.a, int((kb_begin + i) * BK), int(row0), bar_f + 8 * st);
                if (++st == n_st) { st = 0; ph ^= 1; }
            }
        }
        __syncwarp();  // the idle lanes wait here, so that the warp reaches the block barriers converged
    } else if (warp == 2) {
        // The activations' loader (they come from L2: every block reads the same rows).
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t c = 0, ph = 1;
            for (uint32_t i = 0; i < nkb; i++) {
                ok = wait_or_abort(bar_bempty + 8 * c, ph, abort_flag);
                if (!ok) break;
                PROBE(3, i);
                mbar_expect_tx(bar_bfull + 8 * c, b_bytes);
                tma_load_2d(stage_b(c), &maps.b, int((kb_begin + i) * BK), 0, bar_bfull + 8 * c);
                if (++c == CB) { c = 0; ph ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // The MMA issuer. The whole warp runs the loop and one elected lane issues: descriptors and
        // addresses then stay warp-uniform values instead of being moved over for every instruction.
        const uint32_t leader = elect_one();
        const uint32_t idesc = instr_desc(BM, n_pad);
        // A descriptor's low word holds (address >> 4); the stages and the four 32-byte k steps of a
        // stage differ only there.
        const uint64_t da0 = smem_desc(stage_a(0)), db0 = smem_desc(stage_b(0));
        const uint32_t hi_a = uint32_t(da0 >> 32), hi_b = uint32_t(db0 >> 32), lo_a0 = uint32_t(da0), lo_b0 = uint32_t(db0);
        const uint32_t ta0 = tmem_base + a.tmem_a0;
        uint32_t ca = 0, pa = 0, cb = 0, pb = 0;
        for (uint32_t i = 0; i < nkb; i++) {
            ok = wait_or_abort(bar_afull + 8 * ca, pa, abort_flag);
            if (leader) PROBE(4, i);
            ok = ok && wait_or_abort(bar_bfull + 8 * cb, pb, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (leader) PROBE(5, i);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lo_a = lo_a0 + ca * (a_bytes >> 4), lo_b = lo_b0 + cb * (b_bytes >> 4), ta = ta0 + 32 * ca;
            if (leader) {
#pragma unroll
                for (uint32_t k4 = 0; k4 < BK / 16; k4++) {
                    if (INT8) mma_f16_ts(tmem_base, ta + 8 * k4, (uint64_t(hi_b) << 32) | (lo_b + 2 * k4), idesc, (i | k4) != 0 ? 1u : 0u);
                    else mma_f16(tmem_base, (uint64_t(hi_a) << 32) | (lo_a + 2 * k4), (uint64_t(hi_b) << 32) | (lo_b + 2 * k4), idesc, (i | k4) != 0 ? 1u : 0u);
                }
                mma_commit(bar_aempty + 8 * ca);  // arrive once these MMAs have read the stages
                mma_commit(bar_bempty + 8 * cb);
                PROBE(6, i);
            }
            __syncwarp();
            if (++ca == CA) { ca = 0; pa ^= 1; }
            if (++cb == CB) { cb = 0; pb ^= 1; }
        }
        if (ok && leader) mma_commit(bar_accum);
        __syncwarp();
    } else if (INT8) {
        // Raw int8 [128][64] to bf16 in tensor memory. A thread owns a row (the TMEM lane its warp can reach:
        // 32 (warp % 4) + lane), converts its 64 bytes exactly and stores 32 columns of bf16 pairs. The raw
        // tile was swizzled by the TMA (64-byte mode: 16-byte chunk ^= (row >> 1) & 3), which keeps the
        // row-per-thread loads off each other's banks. Groups of four warps take k blocks in turn: a k
        // block's wait -> load -> convert -> store -> arrive chain is long, and this overlaps several of them.
        const uint32_t grp = (warp - FIRST_CONV) / CONV_WPG, quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t row_off = row * 64, sw = (row >> 1) & 3, lane_base = tmem_base + ((quarter * 32) << 16) + a.tmem_a0;
        uint32_t r = grp % R, rph = (grp / R) & 1, c = grp % CA, cph = ((grp / CA) & 1) ^ 1;
        // Scale groups along k (powers of two from 8; the reference's own int8 files: 64, and 8 for the head): a group's scale
        // goes onto its weights here, q * s rounded once to bf16 (the reference multiplies in fp32: this adds what a bf16
        // weight file's rounding adds); one scale per row goes onto the sums in the epilogue, exactly.
        const bool grouped = a.m.group < a.m.k;
        const uint32_t gshift = 31 - __clz(max(a.m.group, 1u));
        const uint16_t* row_scales = grouped ? a.m.scales + size_t(row0 + row) * (a.m.k >> gshift) : nullptr;
        for (uint32_t i = grp; i < nkb; i += CONV_GROUPS) {
            uint32_t sc8[8];  // the scale (twice, as a bf16 pair) of elements 8 e .. 8 e + 7 of this row's k block
            if (grouped) {
#pragma unroll
                for (uint32_t e = 0; e < 8; e++) {
                    const uint32_t sv = __ldg(row_scales + (((kb_begin + i) * BK + 8 * e) >> gshift));
                    sc8[e] = sv | (sv << 16);
                }
            }
            ok = wait_or_abort(bar_rfull + 8 * r, rph, abort_flag) && wait_or_abort(bar_aempty + 8 * c, cph, abort_flag);
            if (!ok) break;
            if (lane == 0 && quarter == 3) PROBE(1, i);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");  // the MMAs that read this stage last are done
            const uint32_t src = stage_raw(r) + row_off;
            uint32_t v[32];
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) {
                uint4 raw;
                asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "r"(src + ((j ^ sw) << 4)));
                cvt_i8x4(raw.x, v[8 * j + 0], v[8 * j + 1]);
                cvt_i8x4(raw.y, v[8 * j + 2], v[8 * j + 3]);
                cvt_i8x4(raw.z, v[8 * j + 4], v[8 * j + 5]);
                cvt_i8x4(raw.w, v[8 * j + 6], v[8 * j + 7]);
            }
            if (grouped) {
#pragma unroll
                for (uint32_t j = 0; j < 32; j++) asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v[j]) : "r"(sc8[j / 4]));
            }
            tmem_st32(lane_base + 32 * c, v);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0 && quarter == 3) PROBE(2, i);
            if (lane == 0) {  // one arrival per warp: an arrival per thread would serialise on the barrier
                mbar_arrive(bar_afull + 8 * c);
                mbar_arrive(bar_rempty + 8 * r);
            }
            for (r += CONV_GROUPS; r >= R; r -= R) rph ^= 1;
            for (c += CONV_GROUPS; c >= CA; c -= CA) cph ^= 1;
        }
    }

    const MatArgs& m = a.m;
    const uint32_t ew = warp - FIRST_CONV;

    // One row's 16 consecutive tokens to global memory (kept small and specialised per epilogue: the
    // code of a fat, fully unrolled epilogue does not stay in the instruction cache). The residual's
    // loads go out together before the first store (it may alias the output); 1/rms comes from
    // shared memory.
    auto emit = [&](uint32_t r, bool valid, uint32_t t0, float scale, auto& v) {  // v: 16 or 8 consecutive tokens of row r
        constexpr uint32_t NTOK = sizeof(v) / sizeof(float);
        const uint32_t row = row0 + r;
        if constexpr (EPI == EPI_QKV) {
            // The row is feature `row` of the qkv projection: dim d of a q, k or v head (whole heads per 64 rows, so
            // a warp's 32 rows are of one kind). RoPE pairs are neighbouring rows, i.e. neighbouring lanes.
            const QkvEpilogue& qe = m.q;
            const uint32_t head = row / 64, d = row % 64, odd = lane & 1;
            const uint32_t kind = head < qe.n_heads ? 0u : head < qe.n_heads + qe.kv.n_kv ? 1u : 2u;  // q, k, v
            const uint32_t psize = 1u << qe.kv.page_shift;
            float x[NTOK];
            float2 cs[NTOK];
#pragma unroll
            for (uint32_t j = 0; j < NTOK; j++) {
                x[j] = (v[j] * scale) * inv_s[t0 + j];
                cs[j] = kind < 2 ? reinterpret_cast<const float2*>(qe.rope)[size_t(pos_s[t0 + j]) * 32 + d / 2] : make_float2(1.0f, 0.0f);
            }
#pragma unroll
            for (uint32_t j = 0; j < NTOK; j++) {
                const float other = __shfl_xor_sync(0xffffffffu, x[j], 1);
                float y = x[j];
                if (kind < 2) {  // (cos a + sin b, cos b - sin a) for the pair (a, b): kernels.metal:727-736
                    const float mine = __fmul_rn(cs[j].x, x[j]), cross = __fmul_rn(cs[j].y, other);
                    y = odd ? __fsub_rn(mine, cross) : __fadd_rn(mine, cross);
                    if (kind == 0) y = __fmul_rn(y, qe.scale_log2);
                }
                const uint32_t bits = f32_to_bf16(y), pair = bits | (__shfl_xor_sync(0xffffffffu, bits, 1) << 16);
                const uint32_t t = t0 + j;
                if (!valid || odd || t >= m.n) continue;  // the even lane writes the pair
                if (kind == 0) {
                    *reinterpret_cast<uint32_t*>(qe.q_b + (size_t(t) * qe.n_heads + head) * 64 + d) = pair;
                } else if (kvrow_s[t] != NO_TOK) {
                    const uint32_t g = kind == 1 ? head - qe.n_heads : head - qe.n_heads - qe.kv.n_kv;
                    uint16_t* cache = kind == 1 ? qe.k_cache : qe.v_cache;
                    *reinterpret_cast<uint32_t*>(cache + (size_t(kvrow_s[t]) + size_t(g) * psize) * 64 + d) = pair;
                }
            }
            return;
        }
        // Loads first, then the arithmetic, then the stores: in that order the tokens overlap.
        float base[NTOK], inv[NTOK], y[NTOK];
#pragma unroll
        for (uint32_t j = 0; j < NTOK; j++) {
            inv[j] = inv_s[t0 + j];
            base[j] = (EPI == EPI_RESID && m.base && valid && t0 + j < m.n) ? m.base[size_t(t0 + j) * m.m + row] : 0.0f;  // (no base: the sum alone, for its bf16 copy and sums of squares)
        }
#pragma unroll
        for (uint32_t j = 0; j < NTOK; j++) {
            const float x = v[j] * scale;
            if (EPI == EPI_SWIGLU) {
                const float other = __shfl_xor_sync(0xffffffffu, x, 1);
                const float gt = x * inv[j], up = other * inv[j];
                y[j] = gt * __fdividef(1.0f, 1.0f + __expf(-gt)) * up;
            } else if (EPI == EPI_NORM) y[j] = x * inv[j] * m.scale;
            else if (EPI == EPI_RESID) y[j] = m.ra * base[j] + m.rb * (m.scale * x);  // (1, 1, 1 for a plain decoder: the same bits as base + x)
            else if (EPI == EPI_HEAD) y[j] = row < m.vocab_real ? x * inv[j] : -INFINITY;
            else if (EPI == EPI_HEAD_CAP) y[j] = row < m.vocab_real ? 23.0f * (1.0f / (1.0f + __expf(-(x + 5.0f) / 7.5f))) : -INFINITY;  // kernels.metal:196-199
            else y[j] = x;
        }
        if (EPI == EPI_RESID && m.ssq_out) {
            // sum(y^2) over the warp's 32 rows for each of the NTOK tokens: a halving butterfly (lanes trade the half of the
            // tokens they give up), a fixed tree, so the sums are the same on every run; then the last two levels in place.
            float w[NTOK];
#pragma unroll
            for (uint32_t j = 0; j < NTOK; j++) w[j] = valid ? y[j] * y[j] : 0.0f;
            uint32_t tk = 0;  // the token (offset in the item) this lane ends up holding
#pragma unroll
            for (uint32_t width = NTOK / 2, bit = 16; width >= 1; width /= 2, bit /= 2) {
                const bool upper = (lane & bit) != 0;
#pragma unroll
                for (uint32_t j = 0; j < width; j++) {
                    const float give = upper ? w[j] : w[j + width], keep = upper ? w[j + width] : w[j];
                    w[j] = keep + __shfl_xor_sync(0xffffffffu, give, bit);
                }
                tk = 2 * tk + (upper ? 1 : 0);
            }
#pragma unroll
            for (uint32_t bit = 16 / NTOK; bit >= 1; bit /= 2) w[0] += __shfl_xor_sync(0xffffffffu, w[0], bit);
            if ((lane & (32 / NTOK - 1)) == 0) ssq_s[(r / 32) * n_pad + t0 + tk] = w[0];
        }
        const bool writes = valid && (EPI != EPI_SWIGLU || (lane & 1) == 0);
        const uint32_t out_w = EPI == EPI_SWIGLU ? m.m / 2 : m.m, out_r = EPI == EPI_SWIGLU ? row / 2 : row;
        if (writes) {
#pragma unroll
            for (uint32_t j = 0; j < NTOK; j++)
                if (t0 + j < m.n) {
                    const size_t o = size_t(t0 + j) * out_w + out_r;
                    if (m.Y) m.Y[o] = y[j];
                    if (m.Yb) m.Yb[o] = f32_to_bf16(y[j]);
                }
        }
    };

    // After a block's emits: its tokens' sums of y^2 over the tile's four row groups, added in order, to global memory.
    auto write_ssq = [&](uint32_t t_lo, uint32_t t_hi) {
        asm volatile("bar.sync 1, %0;" ::"n"(32 * CONV_WARPS) : "memory");  // every epilogue warp, whatever happened before: the row groups' sums are in
        if (*abort_flag) return;
        for (uint32_t t = t_lo + tid - FIRST_CONV * 32; t < t_hi && t < m.n; t += 32 * CONV_WARPS)
            m.ssq_out[size_t(tile) * m.ssq_stride + t] = ((ssq_s[t] + ssq_s[n_pad + t]) + ssq_s[2 * n_pad + t]) + ssq_s[3 * n_pad + t];
    };

    if (warp >= FIRST_CONV) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (uint32_t t = tid - FIRST_CONV * 32; t < n_pad; t += 32 * CONV_WARPS) {
            float inv = 1.0f;
            if (t < a.m.n) {
                if (a.m.inv_in) inv = a.m.inv_in[t];
                else if (a.m.ssq_in) {  // the tiles' sums in tile order
                    float ss = 0.0f;
                    for (uint32_t tl = 0; tl < a.m.ssq_tiles; tl++) ss += a.m.ssq_in[size_t(tl) * a.m.ssq_stride + t];
                    inv = rsqrtf(ss / float(a.m.k) + a.m.eps);
                }
            }
            inv_s[t] = inv;
            if (EPI == EPI_QKV) {
                const QkvEpilogue& qe = a.m.q;
                uint32_t pos = 0, kvrow = NO_TOK;
                if (t < a.m.n) {
                    const uint32_t slot = qe.meta[2 * t], row = qe.tin[2 * t + 1];
                    pos = qe.meta[2 * t + 1];
                    // (the run's first token may lie before this launch's block of tokens: a signed index)
                    const uint32_t cp = qe.cpos ? qe.cpos[t] : qe.meta[2 * (int(t) - int(row)) + 1] + row;  // kernels.metal:74-77 `cache_pos`
                    if (cp != NO_TOK) {
                        const uint32_t page = qe.page_table[size_t(slot) * qe.kv.max_pages + (cp >> qe.kv.page_shift)], psize = 1u << qe.kv.page_shift;
                        kvrow = ((qe.layer * qe.kv.n_pages + page) * qe.kv.n_kv) * psize + (cp & (psize - 1));
                    }
                }
                pos_s[t] = pos;
                kvrow_s[t] = kvrow;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * CONV_WARPS) : "memory");  // the epilogue warps only
        if (tid == FIRST_CONV * 32) PROBE(7, 0);
        if (ok) ok = wait_or_abort(bar_accum, 0, abort_flag);
        if (tid == FIRST_CONV * 32) PROBE(7, 1);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // The warps that share a quarter of the TMEM lanes (rows) take groups of 16 tokens in turn.
            const uint32_t quarter = warp & 3, half = ew >> 2, r = quarter * 32 + lane;
            const float scale = INT8 && m.group >= m.k ? bf16_to_f32(__ldg(m.scales + row0 + r)) : 1.0f;  // (scale groups went onto the weights)
            if (splits == 1) {  // no other block adds to this tile: straight out
                for (uint32_t c0 = 16 * half; c0 < n_pad; c0 += 16 * (CONV_WARPS / 4)) {
                    float acc[16];
                    tmem_ld16(tmem_base + ((quarter * 32) << 16) + c0, acc);
                    emit(r, true, c0, scale, acc);
                }
            }
        }
        if (EPI == EPI_RESID && m.ssq_out && splits == 1) write_ssq(0, n_pad);
    }
    if (!ok) {
        *abort_flag = 1;
        atomicExch(a.err_flag, 2u);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == FIRST_CONV * 32) PROBE(7, 2);
    if (splits > 1) {
        // Split k: the cluster's blocks share out the tile's groups of 16 tokens. Every block sends each group
        // of its partial tile to the block that finishes it -- stores into that block's shared memory, which
        // unlike loads from it wait for no round trip, 128 contiguous bytes per warp (a lane is a row, the
        // buffer is [source rank][group][token][row]) -- and then adds up, in rank order (deterministic), what
        // it was sent. The buffer reuses the rings, so the first cluster barrier says "my MMAs are done, my
        // rings may be written"; after the second nobody touches another block's shared memory again.
        const uint32_t chunks = n_pad / 16, qc = chunks / splits, remc = chunks % splits, slot = qc + 1;
        cluster_sync();
        if (tid == FIRST_CONV * 32) PROBE(7, 3);
        if (warp >= FIRST_CONV && !*abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t quarter = warp & 3, half = ew >> 2, r = quarter * 32 + lane;
            for (uint32_t ch = half; ch < chunks; ch += CONV_WARPS / 4) {
                float acc[16];
                tmem_ld16(tmem_base + ((quarter * 32) << 16) + 16 * ch, acc);
                uint32_t owner, lc;
                if (ch < remc * (qc + 1)) { owner = ch / (qc + 1); lc = ch % (qc + 1); }
                else { owner = remc + (ch - remc * (qc + 1)) / qc; lc = (ch - remc * (qc + 1)) % qc; }
                const uint32_t dst = map_to_rank(smem_base + (((rank * slot + lc) * 16) * BM + r) * 4, owner);
#pragma unroll
                for (uint32_t j = 0; j < 16; j++) asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + j * BM * 4), "f"(acc[j]) : "memory");
            }
        }
        if (tid == FIRST_CONV * 32) PROBE(7, 4);
        cluster_sync();  // every partial is where it will be added up
        if (warp >= FIRST_CONV && !*abort_flag) {
            const float* buf = reinterpret_cast<const float*>(smem);
            const uint32_t ch_begin = rank * qc + min(rank, remc), ch_count = qc + (rank < remc ? 1 : 0);
            // An item: 32 rows x 8 tokens (half a group), so that two groups a block already keep all its warps busy.
            for (uint32_t item = ew; item < ch_count * 2 * (BM / 32); item += CONV_WARPS) {
                const uint32_t lc = item / (2 * (BM / 32)), hf = (item / (BM / 32)) & 1, r = 32 * (item % (BM / 32)) + lane;
                const float scale = INT8 && m.group >= m.k ? bf16_to_f32(__ldg(m.scales + row0 + r)) : 1.0f;  // (scale groups went onto the weights)
                float v[8];
#pragma unroll
                for (uint32_t j = 0; j < 8; j++) v[j] = 0.0f;
                for (uint32_t sr = 0; sr < splits; sr++) {
                    const float* src = buf + size_t((sr * slot + lc) * 16 + 8 * hf) * BM + r;
#pragma unroll
                    for (uint32_t j = 0; j < 8; j++) v[j] += src[j * BM];
                }
                emit(r, true, 16 * (ch_begin + lc) + 8 * hf, scale, v);
            }
        }
        if (EPI == EPI_RESID && m.ssq_out && warp >= FIRST_CONV) {
            const uint32_t ch_begin = rank * qc + min(rank, remc), ch_count = qc + (rank < remc ? 1 : 0);
            write_ssq(16 * ch_begin, 16 * (ch_begin + ch_count));
        }
    }
    if (tid == FIRST_CONV * 32) PROBE(7, 5);
    __syncthreads();
    if (tid == FIRST_CONV * 32) PROBE(7, 6);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

}  // namespace gemm

// Tensor maps are made once per (operand pointer, shape) and kept: the engine's buffers never move.
struct GemmMapCache {
    std::map<std::tuple<const void*, const void*, uint32_t, uint32_t, uint32_t>, gemm::Maps> maps;
};

typedef void (*GemmEntry)(const gemm::Maps, const gemm::Args);
static GemmEntry gemm_entry(bool int8, uint32_t epi, bool paired = false) {
    if (paired) return gemm::gemm_kernel<true, EPI_HEAD, 8>;  // the only shape that runs in waves
    switch (epi) {
    case EPI_NORM: return int8 ? gemm::gemm_kernel<true, EPI_NORM> : gemm::gemm_kernel<false, EPI_NORM>;
    case EPI_RESID: return int8 ? gemm::gemm_kernel<true, EPI_RESID> : gemm::gemm_kernel<false, EPI_RESID>;
    case EPI_SWIGLU: return int8 ? gemm::gemm_kernel<true, EPI_SWIGLU> : gemm::gemm_kernel<false, EPI_SWIGLU>;
    case EPI_HEAD: return int8 ? gemm::gemm_kernel<true, EPI_HEAD> : gemm::gemm_kernel<false, EPI_HEAD>;
    case EPI_QKV: return int8 ? gemm::gemm_kernel<true, EPI_QKV> : gemm::gemm_kernel<false, EPI_QKV>;
    case EPI_HEAD_CAP: return int8 ? gemm::gemm_kernel<true, EPI_HEAD_CAP> : gemm::gemm_kernel<false, EPI_HEAD_CAP>;
    default: return int8 ? gemm::gemm_kernel<true, EPI_RAW> : gemm::gemm_kernel<false, EPI_RAW>;
    }
}

bool gemm_supported(const MatArgs& a) {
    const bool grouped = a.int8 && a.group < a.k;  // scale groups: powers of two from 8
    return a.n >= 1 && a.n <= 256 && a.m % gemm::BM == 0 && a.k % gemm::BK == 0 && (!grouped || (a.group >= 8 && !(a.group & (a.group - 1)))) && a.Xb != nullptr &&
           (a.epi == EPI_RESID || a.epi == EPI_RAW || a.epi == EPI_HEAD_CAP || a.inv_in != nullptr || a.ssq_in != nullptr);
}

void launch_gemm(const MatArgs& a, uint32_t sm_count, uint32_t* err_flag, cudaStream_t s, bool allow_paired) {
    static thread_local GemmMapCache cache;
    static PerDevice configured;
    const uint32_t n_pad = (a.n + 15) / 16 * 16;
    auto key = std::make_tuple(static_cast<const void*>(a.W), static_cast<const void*>(a.Xb), a.m, a.k, n_pad);
    auto it = cache.maps.find(key);
    if (it == cache.maps.end()) {
        gemm::Maps m;
        if (a.int8) make_tensor_map_2d(m.a, a.W, a.k, a.m, gemm::BK, gemm::BM, 1, false, true);
        else make_tensor_map_2d(m.a, a.W, a.k, a.m, gemm::BK, gemm::BM, 2, true);
        make_tensor_map_2d(m.b, a.Xb, a.k, n_pad, gemm::BK, n_pad, 2, true);
        it = cache.maps.emplace(key, m).first;
    }
    // Shared memory: B stages of n_pad x 128 B; bf16 weights, as many A stages of 16 KiB; int8 weights, A
    // stages in tensor memory behind the accumulator and raw stages of 8 KiB in the shared memory left.
    const uint32_t a_bytes = gemm::BM * gemm::BK * 2, b_bytes = n_pad * gemm::BK * 2, raw_bytes = gemm::BM * gemm::BK;
    const uint32_t tiles = a.m / gemm::BM, nkb = a.k / gemm::BK;
    const uint32_t tmem_a0 = (n_pad + 31) / 32 * 32;
    // Several waves of tiles (the head over the vocabulary): two smaller blocks per SM, see threads_of. Each gets half the
    // tensor memory (the accumulator and three A stages in 256 columns) and half the shared memory.
    const bool paired = a.int8 && a.epi == EPI_HEAD && tiles > sm_count && tmem_a0 + 3 * 32 <= 256 && allow_paired;
    const uint32_t budget = paired ? 100 * 1024 : 208 * 1024;
    uint32_t stages_a, stages_b, raw_stages = 0;
    if (a.int8) {
        stages_a = paired ? 3u : std::min(8u, (512 - tmem_a0) / 32);
        stages_b = paired ? 2u : std::max(2u, std::min(4u, (budget - 4 * raw_bytes) / b_bytes));
        raw_stages = std::max(2u, std::min(16u, (budget - stages_b * b_bytes) / raw_bytes));
    } else {
        stages_a = stages_b = std::max(2u, std::min(8u, budget / (a_bytes + b_bytes)));
    }
    const uint32_t ring = paired ? stages_b * b_bytes + raw_stages * raw_bytes
                                 : std::max((a.int8 ? 0 : stages_a * a_bytes) + stages_b * b_bytes + raw_stages * raw_bytes,
                                            (n_pad / 16 + 8) * 16 * gemm::BM * 4);  // the split-k exchange buffer at its largest (8 splits)
    // Unpaired, at least half an SM's shared memory: one block per SM, so that a block never waits for tensor memory
    // behind another one (blocks of different clusters waiting on each other's SMs could deadlock). Paired blocks are in
    // no cluster, and two of them hold exactly an SM's tensor memory.
    const size_t need = size_t(ring) + 1024 + (2 * stages_a + 2 * stages_b + 2 * raw_stages + 1) * 8 + 16 + n_pad * 28;
    const size_t smem = paired ? need : std::max<size_t>(need, 116 * 1024);
    configured.once([] {
        for (int i8 = 0; i8 < 2; i8++)
            for (uint32_t epi = EPI_NORM; epi <= EPI_HEAD_CAP; epi++) VLT_CUDA(cudaFuncSetAttribute(gemm_entry(i8 != 0, epi), cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        VLT_CUDA(cudaFuncSetAttribute(gemm_entry(true, EPI_HEAD, true), cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        VLT_CUDA(cudaFuncSetAttribute(gemm_entry(true, EPI_HEAD, true), cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    });
    // Split k over a cluster when the tiles alone cannot fill the SMs (the reference splits K the
    // same way when a GEMM has few tiles, encode.rs:545-553).
    static thread_local std::map<std::tuple<bool, uint32_t, uint32_t>, uint32_t> wave;  // (int8, smem, cluster size) -> clusters one wave holds
    uint32_t splits = std::max(1u, std::min(8u, std::min(sm_count / tiles, nkb)));  // (1 for a paired launch: more tiles than SMs)
    for (; splits > 1; splits--) {
        auto wk = std::make_tuple(a.int8, uint32_t(smem) * 8 + a.epi, splits);
        auto w = wave.find(wk);
        if (w == wave.end()) {
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3(tiles * splits);
            q.blockDim = dim3(gemm::threads_of(16));
            q.dynamicSmemBytes = smem;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = splits;
            qa[0].val.clusterDim.y = qa[0].val.clusterDim.z = 1;
            q.attrs = qa;
            q.numAttrs = 1;
            int n_clusters = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n_clusters, gemm_entry(a.int8, a.epi), &q);
            w = wave.emplace(wk, e == cudaSuccess ? uint32_t(n_clusters) : 0u).first;
        }
        if (tiles <= w->second) break;  // every cluster is resident at once
    }
    gemm::Args g;
    g.m = a;
    g.n_pad = n_pad;
    g.stages_a = stages_a;
    g.stages_b = stages_b;
    g.raw_stages = raw_stages;
    uint32_t cols = 32;
    while (cols < (a.int8 ? tmem_a0 + 32 * stages_a : n_pad)) cols *= 2;
    g.tmem_cols = cols;
    g.tmem_a0 = tmem_a0;
    g.splits = splits;
    g.err_flag = err_flag;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * splits);
    cfg.blockDim = dim3(gemm::threads_of(paired ? 8 : 16));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the kernel before it drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = splits > 1 ? 2 : 1;
    VLT_CUDA(cudaLaunchKernelEx(&cfg, gemm_entry(a.int8, a.epi, paired), it->second, g));
    launch_counter()++;
#ifdef VLT_GEMM_PROBE
    if (getenv("VLT_GEMM_PROBE")) {
        cudaStreamSynchronize(s);
        static unsigned long long h[8][64];
        cudaMemcpyFromSymbol(h, gemm::g_probe, sizeof(h));
        fprintf(stderr, "gemm m=%u k=%u n=%u splits=%u stages a %u b %u raw %u\n", a.m, a.k, a.n, splits, stages_a, stages_b, raw_stages);
        const unsigned long long t0 = h[0][0];
        fprintf(stderr, "epilogue (ns from the first weight load): starts %lld accumulator done %lld dumped %lld cluster barrier %lld summed %lld emitted %lld left %lld\n",
                (long long)(h[7][0] - t0), (long long)(h[7][1] - t0), (long long)(h[7][2] - t0), (long long)(h[7][3] - t0), (long long)(h[7][4] - t0), (long long)(h[7][5] - t0), (long long)(h[7][6] - t0));
        for (uint32_t i = 0; i < std::min(64u, nkb / splits); i++)
            fprintf(stderr, "kb %2u: tmaA %6lld convstart %6lld convdone %6lld tmaB %6lld afull %6lld bfull %6lld commit %6lld\n", i, (long long)(h[0][i] - t0),
                    (long long)(h[1][i] - t0), (long long)(h[2][i] - t0), (long long)(h[3][i] - t0), (long long)(h[4][i] - t0), (long long)(h[5][i] - t0), (long long)(h[6][i] - t0));
    }
#endif
}

}  // namespace vlt
