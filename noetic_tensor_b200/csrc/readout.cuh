// Readout-fused row statistics: logits = hidden [rows, d] · W [d, V] on the tensor cores, reduced
// to the per-row quantities of the row forward (maximum, log-sum-exp, entropy sum, the given
// token's logit) while the accumulators are still in tensor memory. The [rows, V] logits are
// never written (an optional bf16 copy exists for comparisons).
//
// What it replaces: `Decoder::head` (src/nn/decoder.rs:270-273, a `Linear` x · W with W held as
// [in, out], src/nn/linear.rs:1-3, 51-58) run as `hgemm_bf16_f32acc` (src/tensor/cuda/half_gemm.rs:
// 32-168: bf16 operands, f32 accumulators, 64×64 tiles of mma.sync.m16n8k16) followed by
// token_log_probs / categorical_entropy on the logits it wrote (src/nn/rl.rs:134-141, 405-414).
//
// Shape of the kernel (sm_100a only):
//   - a CTA owns 128 consecutive rows and a contiguous range of 256-column vocabulary tiles;
//   - one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast) of a
//     [128 × 64] tile of the hidden states and a [64 × 256] tile of W per pipeline stage, four
//     stages deep, completion signalled on mbarriers by byte count;
//   - one thread issues tcgen05.mma (M 128, N 256, K 16, bf16 → f32) from shared-memory
//     descriptors into one of two 256-column accumulators in tensor memory, and
//     tcgen05.commit hands finished stages back to the loader and finished tiles to the epilogue;
//   - four epilogue warps read a finished accumulator with tcgen05.ld (thread = row, 32 columns
//     at a time) and fold it into the row's running (m, S = Σe, W = Σe·(z − m)) in column order
//     while the next tile's products run into the other accumulator.
// A row's result over the CTA's column range goes to scratch; a second small kernel merges the
// ranges in index order in f64 (the row kernels' finalisation) and writes the outputs. Every sum
// has a fixed order: results are bitwise reproducible.
//
// Every wait (mbarrier) is bounded by a clock: after kWaitLimitNs without progress a role stops,
// raises the CTA's abort flag (the other roles see it at their next wait), the loader waits,
// again bounded, for its copies in flight, tensor memory is released and the rows of the CTA get
// status bit 2 ("gave up"). Nothing spins forever.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace nrl {

constexpr int kRoBM = 128;       // rows per CTA = lanes of tensor memory
constexpr int kRoBN = 256;       // vocabulary columns per tile = N of one tcgen05.mma
constexpr int kRoBK = 64;        // bf16 elements of K per stage = one 128-byte swizzle row
constexpr int kRoStages = 4;
constexpr int kRoThreads = 192;  // warp 0: loader, warp 1: mma + tensor-memory owner, warps 2-5: epilogue
constexpr uint32_t kRoABytes = kRoBM * kRoBK * 2;  // 16 KB
constexpr uint32_t kRoBBytes = kRoBN * kRoBK * 2;  // 32 KB
constexpr uint32_t kRoStageBytes = kRoABytes + kRoBBytes;
constexpr uint32_t kRoSmemBytes = kRoStages * kRoStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s: far beyond any legitimate wait here
constexpr int kRoPartFloats = 4;  // (m, S, W, token logit) per row and column range

struct ReadoutParams {
    uint64_t rows;
    uint32_t V, d;
    uint32_t tiles;        // ceil(V / 256)
    uint32_t nsplit;       // column ranges per row block
    uint32_t row_blocks;   // ceil(rows / 128)
    uint32_t group_blocks; // row blocks whose CTAs (all column ranges) are launched next to each other
    uint32_t w_is_vd;      // W given as [V, d] (K-major B) instead of [d, V] (N-major B)
    uint32_t round_bf16;   // fold the logits after rounding them to bf16 (what a bf16 logits tensor would hold)
    uint32_t greedy;       // the token is the row's first maximum: its index travels in the part's token-logit slot
    uint32_t allow_bits;   // the allow-mask is one bit per token: u32 words, bit v mod 32 of word v / 32; allow_stride counts words
    float tau;             // temperature: every logit is divided by it (IEEE division, as tempered_logits does) before it is folded
    const int32_t* tokens; // [rows] or null
    float* parts;          // scratch [rows, nsplit, 4]
    uint16_t* logits_out;  // optional bf16 [rows, V]
    // the kernels compiled with EXTRA only:
    const uint8_t* allow;  // optional byte allow-mask [rows, V] or [1, V]
    uint64_t allow_stride; // V or 0
    float2* slog;          // optional sampling log [rows, tiles, 4]: per 64 columns (mass at the running maximum, that maximum)
};
constexpr int kRoLogCols = 64;  // columns per sampling-log entry

// ---- raw PTX wrappers -----------------------------------------------------------------------------
// Bounded wait: false when the CTA aborted or the limit passed (then the abort flag is raised).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 1;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) {
                *abort_flag = 1u;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive f32 columns of this thread's lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
          "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a 128-byte-swizzled tile (version 1, layout type 2), offsets in bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ float round_through_bf16(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x;  // NaN stays NaN
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;  // nearest, ties to even (src/tensor/half.rs:16-27)
    return __uint_as_float(u);
}

// the range of vocabulary tiles of column range `split`
__device__ __forceinline__ void readout_tile_range(const ReadoutParams& p, uint32_t split, uint32_t& t0, uint32_t& t1) {
    const uint32_t per = (p.tiles + p.nsplit - 1) / p.nsplit;
    t0 = min(split * per, p.tiles);
    t1 = min(t0 + per, p.tiles);
}

// One finished 256-column tile of one row (this thread's lane of tensor memory at `taddr`) folded
// into the row's running (m, S, W) at maximum m, and the given token's logit picked up if the
// tile holds it. Columns are taken 32 at a time in index order.
// EXTRA: an allow-mask (excluded columns fold as −FLT_MAX, as in the row kernels) and the sampling log.
template <bool ROUND, bool EXTRA>
__device__ __forceinline__ void readout_fold_tile(const ReadoutParams& p, uint32_t taddr, uint32_t t, uint64_t row, bool live, int32_t tok, float& m, float& S, float& W, float& ztok) {
    float ts = 0.f, tw = 0.f;  // this tile's sums at the running maximum
    float qs = 0.f;            // EXTRA: the current 64 columns' mass at the running maximum
    // EXTRA: the mask bytes of a whole tile inside the vocabulary, 16-byte aligned, are fetched one chunk ahead
    uint4 mq[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    bool mask_fast = false;
    if (EXTRA && p.allow && !p.allow_bits && live) {
        const uint8_t* mp0 = p.allow + row * p.allow_stride + (uint64_t)t * kRoBN;
        mask_fast = (uint64_t)(t + 1) * kRoBN <= p.V && (reinterpret_cast<uintptr_t>(mp0) & 15u) == 0;
        if (mask_fast) {
            mq[0] = ldg_stream16(mp0);
            mq[1] = ldg_stream16(mp0 + 16);
        }
    }
#pragma unroll 1
    for (int c = 0; c < kRoBN / 32; c++) {
        uint32_t r[32];
        tc_ld32(taddr + c * 32, r);
        tc_wait_ld();
        const uint32_t col0 = t * kRoBN + c * 32;
        float z[32];
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float v = __uint_as_float(r[i]);
            if (ROUND) v = round_through_bf16(v);
            z[i] = v;
        }
        if (EXTRA && p.allow && p.allow_bits && live && col0 < p.V) {  // the 32 columns' bits are one word of this row
            const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(p.allow) + row * p.allow_stride + (col0 >> 5));
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (!((word >> i) & 1u)) z[i] = -FLT_MAX;
        } else if (EXTRA && p.allow && live && col0 < p.V) {  // 32 mask bytes of this row: one sector
            const uint8_t* mp = p.allow + row * p.allow_stride + col0;
            if (mask_fast) {
                // this chunk's bytes were loaded one chunk ahead; the next chunk's go out now
                const uint32_t w[8] = {mq[0].x, mq[0].y, mq[0].z, mq[0].w, mq[1].x, mq[1].y, mq[1].z, mq[1].w};
                if (c + 1 < kRoBN / 32) {
                    mq[0] = ldg_stream16(mp + 32);
                    mq[1] = ldg_stream16(mp + 48);
                }
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (((w[i >> 2] >> (8 * (i & 3))) & 0xffu) == 0u) z[i] = -FLT_MAX;
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (col0 + i < p.V && mp[i] == 0) z[i] = -FLT_MAX;
            }
        }
        if (col0 + 32 > p.V) {  // past the vocabulary (TMA filled zeros there): exclude
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (col0 + i >= p.V) z[i] = -FLT_MAX;
        }
        if (p.logits_out && live) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                if (col0 + i + 1 < p.V) {
                    const uint32_t lo = __float_as_uint(round_through_bf16(z[i])) >> 16, hi = __float_as_uint(round_through_bf16(z[i + 1])) & 0xffff0000u;
                    *reinterpret_cast<uint32_t*>(p.logits_out + row * p.V + col0 + i) = lo | hi;
                } else if (col0 + i < p.V) {
                    p.logits_out[row * p.V + col0 + i] = (uint16_t)(__float_as_uint(round_through_bf16(z[i])) >> 16);
                }
            }
        }
        if (p.tau != 1.f) {  // logits / τ (src/nn/rl.rs:475-486); excluded columns stay −FLT_MAX
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (!(z[i] <= -FLT_MAX)) z[i] = __fdiv_rn(z[i], p.tau);
        }
        if (tok >= (int32_t)col0 && tok < (int32_t)(col0 + 32)) {
#pragma unroll
            for (int i = 0; i < 32; i++)
                if ((int32_t)(col0 + i) == tok) ztok = z[i];
        }
        float cm = fmax3_nan(z[0], z[1], z[2]);
#pragma unroll
        for (int i = 3; i < 31; i += 2) cm = fmax3_nan(cm, z[i], z[i + 1]);
        cm = fmax_nan(cm, z[31]);
        cm = fmax_nan(cm, -FLT_MAX);  // a −inf logit is folded as −FLT_MAX: exp underflows to 0 either way and 0·inf cannot appear
        const bool nothing = cm <= -FLT_MAX;  // every column here is excluded (or −inf): no maximum, no mass (a NaN is not "nothing")
        if (!nothing && !(cm <= m)) {  // a new maximum (or a NaN): move the sums
            if (m != NRL_NEG_INF) {
                const float dm = m - cm, sc = expf(dm);
                W = (W + S * dm) * sc;
                S *= sc;
                tw = (tw + ts * dm) * sc;
                ts *= sc;
                if (EXTRA) qs *= sc;
            }
            m = cm;
            if (p.greedy) {  // the first column that holds the new maximum (ties with an earlier chunk never come here)
                uint32_t first = 31u;
#pragma unroll
                for (int i = 30; i >= 0; i--)
                    if (z[i] == cm) first = (uint32_t)i;
                ztok = __uint_as_float(col0 + first);
            }
        }
        // three levels of sums (32 columns, a tile, the range) keep the rounding of the long f32 sums small
        float cs = 0.f, cw = 0.f;
        if (!nothing) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const float tt = fmaxf(z[i], -FLT_MAX) - m;
                const float e = ex2_approx(tt * kLog2e);
                cs += e;
                cw = fmaf(e, tt, cw);
            }
        }
        ts += cs;
        tw += cw;
        if (EXTRA && p.slog) {
            qs = (c & 1) ? qs + cs : cs;
            if ((c & 1) && live) p.slog[(row * p.tiles + t) * (kRoBN / kRoLogCols) + (c >> 1)] = make_float2(qs, m);
        }
    }
    S += ts;
    W += tw;
}

template <bool ROUND, bool EXTRA>
__global__ void __launch_bounds__(kRoThreads, 1) readout_fwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ReadoutParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
    const uint32_t a_base = smem_base, b_base = smem_base + kRoStages * kRoABytes;
    const uint32_t bars = smem_base + kRoStages * kRoStageBytes;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * kRoStages, bar_acc_full = bars + 16 * kRoStages, bar_acc_empty = bar_acc_full + 16, bar_done = bar_acc_empty + 16;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs that run at the same time should share operands in L2: consecutive CTAs cover a group of
    // row blocks (their hidden states stay in L2) times every column range (a range's W tiles are
    // fetched once for the whole group).
    const uint32_t group = blockIdx.x / (p.group_blocks * p.nsplit);
    const uint32_t in_group = min(p.group_blocks, p.row_blocks - group * p.group_blocks);
    const uint32_t within = blockIdx.x - group * p.group_blocks * p.nsplit;
    const uint32_t split = within / in_group, rb = group * p.group_blocks + within % in_group;
    uint32_t t0, t1;
    readout_tile_range(p, split, t0, t1);
    const uint32_t kchunks = (p.d + kRoBK - 1) / kRoBK;

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (int s = 0; s < kRoStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + 8 * a, 1);
            mbar_init(bar_acc_empty + 8 * a, 4);
        }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // the whole warp allocates all 512 columns: two 256-column accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_addr(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---- loader ------------------------------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0, issued = 0;
            bool ok = true;
            for (uint32_t t = t0; t < t1 && ok; t++) {
                for (uint32_t kc = 0; kc < kchunks; kc++, it++) {
                    const uint32_t s = it % kRoStages;
                    if (!mbar_wait(bar_empty + 8 * s, ((it / kRoStages) & 1u) ^ 1u, &abort_flag)) { ok = false; break; }
                    mbar_expect_tx(bar_full + 8 * s, kRoStageBytes);
                    tma_load_2d(a_base + s * kRoABytes, &map_x, (int32_t)(kc * kRoBK), (int32_t)(rb * kRoBM), bar_full + 8 * s);
                    if (p.w_is_vd) {
                        tma_load_2d(b_base + s * kRoBBytes, &map_w, (int32_t)(kc * kRoBK), (int32_t)(t * kRoBN), bar_full + 8 * s);
                    } else {
#pragma unroll
                        for (int j = 0; j < kRoBN / 64; j++)  // W [d, V]: four [64 k × 64 n] boxes, n contiguous
                            tma_load_2d(b_base + s * kRoBBytes + j * (kRoBK * 128), &map_w, (int32_t)(t * kRoBN + j * 64), (int32_t)(kc * kRoBK), bar_full + 8 * s);
                    }
                    issued = it + 1;
                }
            }
            if (!ok || abort_flag) {
                // copies still in flight write this CTA's shared memory: wait for them (bounded) before the CTA may end
                const uint32_t first = issued > (uint32_t)kRoStages ? issued - kRoStages : 0u;
                for (uint32_t j = first; j < issued; j++) {
                    volatile uint32_t never = 0u;
                    mbar_wait(bar_full + 8 * (j % kRoStages), (j / kRoStages) & 1u, &never, 20000000ull);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ---------------------------------------------------------------------
        if (lane == 0) {
            // instruction descriptor: D f32, A and B bf16, A K-major, B K-major ([V, d]) or N-major ([d, V]), N 256, M 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((p.w_is_vd ? 0u : 1u) << 16) | ((uint32_t)(kRoBN >> 3) << 17) | ((uint32_t)(kRoBM >> 4) << 24);
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = t0; t < t1 && ok; t++) {
                const uint32_t n = t - t0, acc = n & 1u;
                if (!mbar_wait(bar_acc_empty + 8 * acc, ((n >> 1) & 1u) ^ 1u, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem + acc * kRoBN;
                for (uint32_t kc = 0; kc < kchunks; kc++, it++) {
                    const uint32_t s = it % kRoStages;
                    if (!mbar_wait(bar_full + 8 * s, (it / kRoStages) & 1u, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = a_base + s * kRoABytes, b_addr = b_base + s * kRoBBytes;
#pragma unroll
                    for (int k = 0; k < kRoBK / 16; k++) {
                        // A, and B as [V, d]: K-major, rows of 128 bytes, groups of 8 rows 1024 bytes apart; 16 elements of K = 32 bytes along the row
                        const uint64_t da = smem_desc_sw128(a_addr + k * 32, 16, 1024);
                        // B as [d, V]: N-major, 64 columns contiguous, column blocks 8 KB apart, groups of 8 k-rows 1024 bytes apart; 16 k-rows = 2048 bytes
                        const uint64_t db = p.w_is_vd ? smem_desc_sw128(b_addr + k * 32, 16, 1024) : smem_desc_sw128(b_addr + k * 2048, kRoBK * 128, 1024);
                        tc_mma_bf16(d_tmem, da, db, idesc, (kc | (uint32_t)k) != 0u);
                    }
                    tc_commit(bar_empty + 8 * s);  // the stage is free once these products have read it
                }
                if (ok) tc_commit(bar_acc_full + 8 * acc);
            }
            // before tensor memory may be released every product issued above must have finished
            tc_commit(bar_done);
        }
    } else {
        // ---- epilogue: thread = row ------------------------------------------------------------------
        const uint32_t quarter = (uint32_t)warp & 3u;  // the 32 lanes of tensor memory this warp may read
        const uint32_t r_in_block = quarter * 32u + (uint32_t)lane;
        const uint64_t row = (uint64_t)rb * kRoBM + r_in_block;
        const bool live = row < p.rows;
        const int32_t tok = (live && p.tokens) ? p.tokens[row] : -1;
        float m = NRL_NEG_INF, S = 0.f, W = 0.f, ztok = __int_as_float(0x7fc00000);  // NaN: "the token is not in this range"
        bool ok = true;
        for (uint32_t t = t0; t < t1 && ok; t++) {
            const uint32_t n = t - t0, acc = n & 1u;
            if (!mbar_wait(bar_acc_full + 8 * acc, (n >> 1) & 1u, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            readout_fold_tile<ROUND, EXTRA>(p, tmem + ((quarter * 32u) << 16) + acc * kRoBN, t, row, live, tok, m, S, W, ztok);
            // this accumulator may be overwritten once all four epilogue warps are done with it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
        }
        if (live) {
            float4 out = make_float4(m, S, W, ztok);
            if (!ok || abort_flag) out = make_float4(0.f, -1.f, 0.f, 0.f);  // S = −1 marks "gave up" for the merge
            reinterpret_cast<float4*>(p.parts)[row * p.nsplit + split] = out;
        }
    }

    // ---- teardown ------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (lane == 0) {
            // all products have finished (on an aborted CTA the wait gives up after 20 ms)
            volatile uint32_t never = 0u;
            mbar_wait(bar_done, 0u, &never, 20000000ull);
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

// ---- the same kernel on CTA pairs (cta_group::2) ---------------------------------------------------
//
// Two CTAs of a cluster, on two SMs, work on one 256-row block: CTA r of the pair owns rows
// 128·r … of it (its hidden-state tiles, its 128 lanes of tensor memory, its epilogue) and loads
// only HALF of each W tile (128 of the 256 columns); one thread of the pair's first CTA issues
// tcgen05.mma.cta_group::2 (M 256, N 256), which reads both CTAs' shared memory and writes both
// CTAs' accumulators. Per unit of tensor work an SM then takes 32 KB instead of 48 KB out of L2,
// and the freed shared memory holds six stages instead of four.
//   loads:     cp.async.bulk.tensor.2d.cta_group::2 (no multicast), every copy of the pair
//              completing on the FIRST CTA's `full` barrier, which expects both CTAs' bytes;
//   hand-back: tcgen05.commit.cta_group::2 … multicast::cluster to the `empty` barriers of both
//              CTAs (each CTA's loader waits on its own) and to both `accumulator full` barriers;
//   epilogue:  both CTAs' epilogue warps arrive on the first CTA's `accumulator empty` barrier
//              (a remote mbarrier arrive for the second CTA).
// Waits are bounded as above; the pair meets at a cluster barrier before either CTA exits.
constexpr int kRoStages2 = 6;  // a seventh stage fits the 227 KB and measured the same
constexpr uint32_t kRoBBytes2 = kRoBBytes / 2;                 // 16 KB: this CTA's half of the W tile
constexpr uint32_t kRoStageBytes2 = kRoABytes + kRoBBytes2;    // 32 KB
constexpr uint32_t kRoSmemBytes2 = kRoStages2 * kRoStageBytes2 + 1024 + 256;
// a shared-memory address of this CTA -> the address of the same offset in the cluster's first CTA
__device__ __forceinline__ uint32_t in_first_cta(uint32_t addr) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(0u));
    return r;
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar_in_first_cta) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y),
                 "r"(bar_in_first_cta)
                 : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {  // arrives on `bar` in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Work items are (256-row block, column range) pairs laid out in groups as above; the grid holds
// `gridDim.x / 2 / (group_blocks · nsplit)` groups' worth of clusters and a cluster walks the groups
// with that stride (one cluster per item when the grid covers every group).
template <bool ROUND, bool EXTRA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kRoThreads, 1)
    readout_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ReadoutParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = smem_base, b_base = smem_base + kRoStages2 * kRoABytes;
    const uint32_t bars = smem_base + kRoStages2 * kRoStageBytes2;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * kRoStages2, bar_acc_full = bars + 16 * kRoStages2, bar_acc_empty = bar_acc_full + 16, bar_done = bar_acc_empty + 16;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0: issues the products; both load and fold
    const uint32_t per_group = p.group_blocks * p.nsplit;  // row_blocks, group_blocks: in 256-row blocks
    const uint32_t cluster = (blockIdx.x >> 1) % per_group, group0 = (blockIdx.x >> 1) / per_group, gstride = max(1u, (gridDim.x >> 1) / per_group);
    const uint32_t ngroups = (p.row_blocks + p.group_blocks - 1) / p.group_blocks;
    const uint32_t kchunks = (p.d + kRoBK - 1) / kRoBK;
    // work item of this cluster in group g: false when the group has fewer items than the wave has clusters
    auto item = [&](uint32_t g, uint32_t& split, uint32_t& rb, uint32_t& t0, uint32_t& t1) -> bool {
        const uint32_t in_group = min(p.group_blocks, p.row_blocks - g * p.group_blocks);
        if (cluster >= in_group * p.nsplit) return false;
        split = cluster / in_group;
        rb = (g * p.group_blocks + cluster % in_group) * 2 + rank;  // this CTA's 128-row block
        readout_tile_range(p, split, t0, t1);
        return true;
    };

    if (threadIdx.x == 0) {
        abort_flag = 0u;
        for (int s = 0; s < kRoStages2; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + 8 * a, 1);
            mbar_init(bar_acc_empty + 8 * a, 8);  // four epilogue warps of each CTA
        }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_addr(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        tc_fence_before();
    }
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anything crosses between them
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---- loader (both CTAs) -------------------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t g = group0; g < ngroups && ok; g += gstride) {
                uint32_t split, rb, t0, t1;
                if (!item(g, split, rb, t0, t1)) continue;
                for (uint32_t t = t0; t < t1 && ok; t++) {
                    for (uint32_t kc = 0; kc < kchunks; kc++, it++) {
                        const uint32_t s = it % kRoStages2;
                        if (!mbar_wait(bar_empty + 8 * s, ((it / kRoStages2) & 1u) ^ 1u, &abort_flag)) { ok = false; break; }
                        const uint32_t full_first = in_first_cta(bar_full + 8 * s);
                        if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * kRoStageBytes2);  // both CTAs' copies land on this barrier
                        tma_load_2d_pair(a_base + s * kRoABytes, &map_x, (int32_t)(kc * kRoBK), (int32_t)(rb * kRoBM), full_first);
                        const uint32_t n0 = t * kRoBN + rank * (kRoBN / 2);  // this CTA's half of the tile's columns
                        if (p.w_is_vd) {
                            tma_load_2d_pair(b_base + s * kRoBBytes2, &map_w, (int32_t)(kc * kRoBK), (int32_t)n0, full_first);
                        } else {
#pragma unroll
                            for (int j = 0; j < kRoBN / 128; j++)
                                tma_load_2d_pair(b_base + s * kRoBBytes2 + j * (kRoBK * 128), &map_w, (int32_t)(n0 + j * 64), (int32_t)(kc * kRoBK), full_first);
                        }
                    }
                }
            }
            if ((!ok || abort_flag) && it) {
                // give this CTA's copies in flight time to land before the pair may end (their completion is
                // counted on the first CTA's barrier, which this CTA cannot wait on by phase: a bounded sleep)
                const unsigned long long t_start = global_ns();
                while (global_ns() - t_start < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue (first CTA only) -------------------------------------------------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((p.w_is_vd ? 0u : 1u) << 16) | ((uint32_t)(kRoBN >> 3) << 17) | ((uint32_t)((2 * kRoBM) >> 4) << 24);
            uint32_t it = 0, n = 0;
            bool ok = true;
            for (uint32_t g = group0; g < ngroups && ok; g += gstride) {
                uint32_t split, rb, t0, t1;
                if (!item(g, split, rb, t0, t1)) continue;
                for (uint32_t t = t0; t < t1 && ok; t++, n++) {
                    const uint32_t acc = n & 1u;
                    if (!mbar_wait(bar_acc_empty + 8 * acc, ((n >> 1) & 1u) ^ 1u, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem + acc * kRoBN;
                    for (uint32_t kc = 0; kc < kchunks; kc++, it++) {
                        const uint32_t s = it % kRoStages2;
                        if (!mbar_wait(bar_full + 8 * s, (it / kRoStages2) & 1u, &abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = a_base + s * kRoABytes, b_addr = b_base + s * kRoBBytes2;
#pragma unroll
                        for (int k = 0; k < kRoBK / 16; k++) {
                            const uint64_t da = smem_desc_sw128(a_addr + k * 32, 16, 1024);
                            const uint64_t db = p.w_is_vd ? smem_desc_sw128(b_addr + k * 32, 16, 1024) : smem_desc_sw128(b_addr + k * 2048, kRoBK * 128, 1024);
                            tc_mma_bf16_pair(d_tmem, da, db, idesc, (kc | (uint32_t)k) != 0u);
                        }
                        tc_commit_pair(bar_empty + 8 * s);
                    }
                    if (ok) tc_commit_pair(bar_acc_full + 8 * acc);
                }
            }
            tc_commit_pair(bar_done);
        }
    } else {
        // ---- epilogue (both CTAs): thread = row ----------------------------------------------------------
        const uint32_t quarter = (uint32_t)warp & 3u;
        const uint32_t r_in_block = quarter * 32u + (uint32_t)lane;
        uint32_t n = 0;
        bool ok = true;
        for (uint32_t g = group0; g < ngroups; g += gstride) {
            uint32_t split, rb, t0, t1;
            if (!item(g, split, rb, t0, t1)) continue;
            const uint64_t row = (uint64_t)rb * kRoBM + r_in_block;
            const bool live = row < p.rows;
            const int32_t tok = (live && p.tokens) ? p.tokens[row] : -1;
            float m = NRL_NEG_INF, S = 0.f, W = 0.f, ztok = __int_as_float(0x7fc00000);
            for (uint32_t t = t0; t < t1 && ok; t++, n++) {
                const uint32_t acc = n & 1u;
                if (!mbar_wait(bar_acc_full + 8 * acc, (n >> 1) & 1u, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                readout_fold_tile<ROUND, EXTRA>(p, tmem + ((quarter * 32u) << 16) + acc * kRoBN, t, row, live, tok, m, S, W, ztok);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(in_first_cta(bar_acc_empty + 8 * acc));
            }
            if (live) {
                float4 out = make_float4(m, S, W, ztok);
                if (!ok || abort_flag) out = make_float4(0.f, -1.f, 0.f, 0.f);  // "gave up": also for the items not reached
                reinterpret_cast<float4*>(p.parts)[row * p.nsplit + split] = out;
            }
        }
    }

    // ---- teardown ------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (lane == 0) {
            volatile uint32_t never = 0u;
            mbar_wait(bar_done, 0u, &never, 20000000ull);  // every product has finished (multicast to both CTAs)
        }
        __syncwarp();
    }
    cluster_sync_all();  // neither CTA leaves while the other may still reach into its shared or tensor memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

// Merge the column ranges of each row in index order (f64, as the row kernels finalise) and write
// the outputs: rowstats (m, ln Z, 0, 0), entropy = ln Z − W / Z, logp = z_tok − m − ln Z.
// `greedy`: tokens is an output, the index kept by the first range (in column order) that reached the row's maximum.
__global__ void readout_finish_kernel(uint64_t rows, uint32_t nsplit, const float* parts, int32_t* tokens, float* logp, float* entropy, float* rowstats, uint8_t* status, uint32_t greedy) {
    const uint64_t row = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const float4* pr = reinterpret_cast<const float4*>(parts) + row * nsplit;
    float m = NRL_NEG_INF;
    for (uint32_t s = 0; s < nsplit; s++) m = fmax_nan(m, pr[s].x);
    double Z = 0.0, Wt = 0.0;
    float ztok = __int_as_float(0x7fc00000);
    for (uint32_t s = 0; s < nsplit; s++) {
        const float4 a = pr[s];
        if (a.x != NRL_NEG_INF && a.y > 0.f) {
            const double dm = (double)a.x - (double)m, c = (double)expf(a.x - m);
            Z += c * (double)a.y;
            Wt += c * ((double)a.z + (double)a.y * dm);
        }
        if (!greedy && a.w == a.w) ztok = a.w;
    }
    int32_t picked = -1;
    if (greedy) {
        for (uint32_t s = 0; s < nsplit && picked < 0; s++)
            if (pr[s].x == m && pr[s].y > 0.f) picked = (int32_t)__float_as_uint(pr[s].w);
        ztok = m;
    }
    uint32_t st = 0u;
    for (uint32_t s = 0; s < nsplit; s++)
        if (pr[s].y < 0.f) st |= 4u;
    if (m != m) st |= 2u;
    else if (m == NRL_NEG_INF || m <= -FLT_MAX) st |= 1u;
    const double lnZ = log(Z);
    if (greedy) tokens[row] = st ? -1 : picked;
    if (st) {
        const float nan = __int_as_float(0x7fc00000);
        if (logp) logp[row] = nan;
        if (entropy) entropy[row] = nan;
        if (rowstats) reinterpret_cast<float4*>(rowstats)[row] = make_float4(nan, nan, nan, nan);
    } else {
        if (rowstats) reinterpret_cast<float4*>(rowstats)[row] = make_float4(m, (float)lnZ, 0.f, 0.f);
        if (entropy) entropy[row] = (float)(lnZ - Wt / Z);
        if (logp && tokens) {
            const int32_t tk = tokens[row];
            // a token outside [0, V) has no logit: NaN; an excluded one (−inf logit) has log-prob −inf
            logp[row] = (ztok != ztok) ? ztok : (ztok <= -FLT_MAX ? NRL_NEG_INF : (ztok - m) - (float)lnZ);
            (void)tk;
        }
    }
    if (status) status[row] = (uint8_t)st;
}

// ---- sampling out of the fused pass -----------------------------------------------------------------
//
// token = min{k : Σ_{v≤k} e_v > u·Z}, as in the row forward. The tensor-core pass leaves, per row
// and per 64 columns, the mass at the maximum the row had reached then. Three small kernels follow:
//   readout_pick_kernel    one warp per row: merge the ranges (the row's m, Z, entropy), rescale the
//                          logged masses to m and find the 64 columns that hold u·Z with warp scans
//                          in index order;
//   readout_bucket_kernel  one block: rows grouped by the 64-column slab they picked (a counting
//                          sort; the order inside a group does not enter any result), so that
//   readout_draw_kernel    one block per slab computes the slab's 64 logits again for every row
//                          that picked it — 64 dot products of length d in f32, lanes over columns —
//                          with the slab of W (64 · d · 2 bytes) coming from HBM once instead of once
//                          per row, applies rounding and mask as the pass did, and walks to the
//                          token. Its log-prob is z_token − m − ln Z with that recomputed logit (it
//                          differs from the tensor cores' accumulation of the same products by the
//                          f32 rounding of a sum of d terms).
struct ReadoutPick {
    double resid;    // u·Z minus the mass before the slab; 1e300: take the slab's last token with mass
    float m, lnZ;
    int32_t slab;    // index of the 64-column slab, −1 for a refused row
    uint32_t pad;
};

__global__ void __launch_bounds__(256) readout_pick_kernel(ReadoutParams p, const float* uniforms, ReadoutPick* picks, int32_t* tokens, float* logp, float* entropy, float* rowstats,
                                                          uint8_t* status) {
    const uint64_t row = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int lane = threadIdx.x & 31;
    const float4* pr = reinterpret_cast<const float4*>(p.parts) + row * p.nsplit;
    float m = NRL_NEG_INF;
    uint32_t st = 0u;
    for (uint32_t s = 0; s < p.nsplit; s++) {
        m = fmax_nan(m, pr[s].x);
        if (pr[s].y < 0.f) st |= 4u;
    }
    double Z = 0.0, Wt = 0.0;
    for (uint32_t s = 0; s < p.nsplit; s++) {
        const float4 a = pr[s];
        if (a.x != NRL_NEG_INF && a.y > 0.f) {
            const double dm = (double)a.x - (double)m, c = (double)expf(a.x - m);
            Z += c * (double)a.y;
            Wt += c * ((double)a.z + (double)a.y * dm);
        }
    }
    if (m != m) st |= 2u;
    else if (m == NRL_NEG_INF || m <= -FLT_MAX) st |= 1u;
    const double lnZ = log(Z);
    const float nan = __int_as_float(0x7fc00000);
    ReadoutPick pk;
    pk.resid = 0.0; pk.m = m; pk.lnZ = (float)lnZ; pk.slab = -1; pk.pad = 0u;
    if (st) {
        if (lane == 0) {
            tokens[row] = -1;
            if (logp) logp[row] = nan;
            if (entropy) entropy[row] = nan;
            if (rowstats) reinterpret_cast<float4*>(rowstats)[row] = make_float4(nan, nan, nan, nan);
            if (status) status[row] = (uint8_t)st;
            picks[row] = pk;
        }
        return;
    }
    const double target = (double)uniforms[row] * Z;
    const uint32_t nlog = p.tiles * (kRoBN / kRoLogCols);
    const float2* lg = p.slog + row * nlog;
    double before = 0.0, run = 0.0;
    int32_t slab = -1, last_mass = -1;
    for (uint32_t e0 = 0; e0 < nlog && slab < 0; e0 += 32) {
        const uint32_t e = e0 + lane;
        double x = 0.0;
        if (e < nlog && (uint64_t)e * kRoLogCols < p.V) {
            const float2 q = lg[e];
            if (q.x > 0.f) x = (double)q.x * (double)expf(q.y - m);
        }
        const double incl = warp_scan_incl(x, lane);
        const uint32_t cross = __ballot_sync(0xffffffffu, x > 0.0 && run + incl > target);
        const uint32_t has = __ballot_sync(0xffffffffu, x > 0.0);
        if (has) last_mass = (int32_t)e0 + 31 - __clz(has);
        if (cross) {
            const int owner = __ffs(cross) - 1;
            slab = (int32_t)e0 + owner;
            before = run + __shfl_sync(0xffffffffu, incl - x, owner);
        }
        run += __shfl_sync(0xffffffffu, incl, 31);
    }
    pk.resid = target - before;
    if (slab < 0) {  // rounding left no crossing: the last slab with mass, its last token with mass
        slab = last_mass;
        pk.resid = 1e300;
    }
    pk.slab = slab;
    if (lane == 0) {
        picks[row] = pk;
        if (rowstats) reinterpret_cast<float4*>(rowstats)[row] = make_float4(m, (float)lnZ, 0.f, 0.f);
        if (entropy) entropy[row] = (float)(lnZ - Wt / Z);
        if (status) status[row] = 0;
    }
}

// Rows grouped by slab: order[bucket_start[s] .. bucket_start[s + 1]) are the rows that picked slab s.
constexpr int kRoMaxSlabs = 8192;  // slabs a single block can count in shared memory (V ≤ 524 288)
__global__ void __launch_bounds__(1024) readout_bucket_kernel(uint64_t rows, uint32_t nslabs, const ReadoutPick* picks, uint32_t* bucket_start, uint32_t* order) {
    __shared__ uint32_t cnt[kRoMaxSlabs];
    __shared__ uint32_t carry;
    for (uint32_t i = threadIdx.x; i < nslabs; i += blockDim.x) cnt[i] = 0u;
    __syncthreads();
    for (uint64_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const int32_t s = picks[r].slab;
        if (s >= 0) atomicAdd(&cnt[s], 1u);  // a count of work items: no result depends on the order of these additions
    }
    __syncthreads();
    // exclusive scan of the counts, 1024 slabs at a time
    if (threadIdx.x == 0) carry = 0u;
    __syncthreads();
    for (uint32_t base = 0; base < nslabs; base += blockDim.x) {
        const uint32_t i = base + threadIdx.x;
        const uint32_t c = i < nslabs ? cnt[i] : 0u;
        // block-wide inclusive scan through shared memory (Hillis-Steele on the warp, then the warps' totals)
        uint32_t x = c;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, x, k);
            if (lane >= k) x += y;
        }
        __shared__ uint32_t wsum[32];
        if (lane == 31) wsum[warp] = x;
        __syncthreads();
        if (warp == 0) {
            uint32_t w = wsum[lane];
#pragma unroll
            for (int k = 1; k < 32; k <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, w, k);
                if (lane >= k) w += y;
            }
            wsum[lane] = w;
        }
        __syncthreads();
        const uint32_t incl = x + (warp ? wsum[warp - 1] : 0u) + carry;
        if (i < nslabs) {
            bucket_start[i] = incl - c;
            cnt[i] = incl - c;  // becomes the slab's fill cursor
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) bucket_start[nslabs] = carry;
    __syncthreads();
    for (uint64_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const int32_t s = picks[r].slab;
        if (s >= 0) order[atomicAdd(&cnt[s], 1u)] = (uint32_t)r;
    }
}

// grid (kRoDrawParts, slabs): the rows that picked slab s are taken kRoDrawRows at a time, block (y, s) taking the
// groups y, y + kRoDrawParts, …; the rows of a group share one pass over the slab of W (64 · d · 2 bytes: with one row
// per pass the kernel was bound by what an SM can pull out of L2). The eight warps split the d terms of the dot
// products (each warp a contiguous eighth, 16 loads of W deep), the partial sums meet in shared memory and are added
// in warp order: a row's recomputed logits do not depend on which rows share its pass. Warp i then walks row i.
constexpr int kRoDrawParts = 8;
constexpr int kRoDrawRows = 4;
__global__ void __launch_bounds__(256) readout_draw_kernel(ReadoutParams p, const ReadoutPick* picks, const uint32_t* bucket_start, const uint32_t* order, int32_t* tokens, float* logp,
                                                          const uint16_t* hidden, const uint16_t* weights) {
    constexpr int R = kRoDrawRows;
    __shared__ float part[8][R][kRoLogCols];
    const uint32_t slab = blockIdx.y;
    const uint32_t r0 = bucket_start[slab], n = bucket_start[slab + 1] - r0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float nan = __int_as_float(0x7fc00000);
    const uint32_t c0 = slab * kRoLogCols, ca = c0 + 2 * lane;  // this lane's two columns
    const uint32_t kper = ((p.d + 63) / 64) * 8;                // terms per warp, a multiple of 8 (as d is)
    const uint32_t k0 = min((uint32_t)warp * kper, p.d), k1 = min(k0 + kper, p.d);
    for (uint32_t g = blockIdx.x * R; g < n; g += gridDim.x * R) {
        const uint32_t cnt = min((uint32_t)R, n - g);
        uint64_t rows[R];
        const uint16_t* x[R];
        float z[R][2];
#pragma unroll
        for (int i = 0; i < R; i++) {
            rows[i] = order[r0 + g + min((uint32_t)i, cnt - 1)];  // a short group repeats its last row: computed, not used
            x[i] = hidden + rows[i] * p.d;
            z[i][0] = z[i][1] = 0.f;
        }
        if (ca < p.V) {
            if (p.w_is_vd) {
                const uint16_t *wa = weights + (uint64_t)ca * p.d, *wb = wa + p.d;
#pragma unroll 2
                for (uint32_t k = k0; k < k1; k += 8) {
                    const uint4 aq = *reinterpret_cast<const uint4*>(wa + k), bq = *reinterpret_cast<const uint4*>(wb + k);
                    const uint32_t aw[4] = {aq.x, aq.y, aq.z, aq.w}, bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
                    for (int i = 0; i < R; i++) {
                        const uint4 xq = *reinterpret_cast<const uint4*>(x[i] + k);
                        const uint32_t xw[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            z[i][0] = fmaf(bf16_lo(xw[t]), bf16_lo(aw[t]), z[i][0]);
                            z[i][0] = fmaf(bf16_hi(xw[t]), bf16_hi(aw[t]), z[i][0]);
                            z[i][1] = fmaf(bf16_lo(xw[t]), bf16_lo(bw[t]), z[i][1]);
                            z[i][1] = fmaf(bf16_hi(xw[t]), bf16_hi(bw[t]), z[i][1]);
                        }
                    }
                }
            } else {
                const uint16_t* wp = weights + ca;
#pragma unroll 2
                for (uint32_t k = k0; k < k1; k += 8) {
                    uint32_t ww[8];
#pragma unroll
                    for (int t = 0; t < 8; t++) ww[t] = *reinterpret_cast<const uint32_t*>(wp + (uint64_t)(k + t) * p.V);
#pragma unroll
                    for (int i = 0; i < R; i++) {
                        const uint4 xq = *reinterpret_cast<const uint4*>(x[i] + k);  // the same address in every lane: one fetch
                        const uint32_t xw[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            const float xl = bf16_lo(xw[t]), xh = bf16_hi(xw[t]);
                            z[i][0] = fmaf(xl, bf16_lo(ww[2 * t]), z[i][0]);
                            z[i][1] = fmaf(xl, bf16_hi(ww[2 * t]), z[i][1]);
                            z[i][0] = fmaf(xh, bf16_lo(ww[2 * t + 1]), z[i][0]);
                            z[i][1] = fmaf(xh, bf16_hi(ww[2 * t + 1]), z[i][1]);
                        }
                    }
                }
            }
        }
        __syncthreads();  // the previous group's readers of `part` are done
#pragma unroll
        for (int i = 0; i < R; i++) {
            part[warp][i][2 * lane] = z[i][0];
            part[warp][i][2 * lane + 1] = z[i][1];
        }
        __syncthreads();
        if ((uint32_t)warp >= cnt) continue;
        uint64_t row = rows[0];
#pragma unroll
        for (int i = 1; i < R; i++)
            if (warp == i) row = rows[i];
        float z0 = part[0][warp][2 * lane], z1 = part[0][warp][2 * lane + 1];
#pragma unroll
        for (int w = 1; w < 8; w++) {
            z0 += part[w][warp][2 * lane];
            z1 += part[w][warp][2 * lane + 1];
        }
        const ReadoutPick pk = picks[row];
        if (p.round_bf16) { z0 = round_through_bf16(z0); z1 = round_through_bf16(z1); }
        if (p.tau != 1.f) { z0 = __fdiv_rn(z0, p.tau); z1 = __fdiv_rn(z1, p.tau); }
        bool ok0 = ca < p.V, ok1 = ca + 1 < p.V;
        if (p.allow && p.allow_bits) {
            const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(p.allow) + row * p.allow_stride + (ca >> 5));
            ok0 = ok0 && ((word >> (ca & 31u)) & 1u);
            ok1 = ok1 && ((word >> ((ca + 1) & 31u)) & 1u);
        } else if (p.allow) {
            const uint8_t* mp = p.allow + row * p.allow_stride;
            ok0 = ok0 && mp[ca] != 0;
            ok1 = ok1 && mp[ca + 1] != 0;
        }
        const float m = pk.m;
        const float e0v = ok0 ? ex2_approx((fmaxf(z0, -FLT_MAX) - m) * kLog2e) : 0.f, e1v = ok1 ? ex2_approx((fmaxf(z1, -FLT_MAX) - m) * kLog2e) : 0.f;
        const double pair = (double)e0v + (double)e1v;
        const double incl = warp_scan_incl(pair, lane);
        const uint32_t cross = __ballot_sync(0xffffffffu, pair > 0.0 && incl > pk.resid);
        const uint32_t has = __ballot_sync(0xffffffffu, pair > 0.0);
        int32_t token = -1;
        float ztok = nan;
        if (has) {
            const int owner = cross ? __ffs(cross) - 1 : 31 - __clz(has);
            int32_t tk = -1;
            float zt = nan;
            if (lane == owner) {
                const double b0 = incl - pair;
                if (cross ? (e0v > 0.f && b0 + (double)e0v > pk.resid) : !(e1v > 0.f)) { tk = (int32_t)ca; zt = z0; }
                else if (e1v > 0.f) { tk = (int32_t)ca + 1; zt = z1; }
                else { tk = (int32_t)ca; zt = z0; }
            }
            token = __shfl_sync(0xffffffffu, tk, owner);
            ztok = __shfl_sync(0xffffffffu, zt, owner);
        }
        if (lane == 0) {
            tokens[row] = token;
            if (logp) logp[row] = token < 0 ? nan : (ztok - m) - pk.lnZ;
        }
    }
}

}  // namespace nrl
