// Row forward: one streaming pass over each vocabulary row computing, per row, the online
// max / log-sum-exp of the tempered, masked logits, the entropy and KL accumulators, and the
// sampled (or given, or greedy) token with its log-probabilities.
//
// Work decomposition (a pure function of rows and V, never of timing or occupancy, so the
// reduction order is fixed and results are bitwise reproducible):
//   row  → `nsplit` blocks, each a contiguous, tile-aligned range of the row (nsplit = 1 when
//          there are enough rows to fill the machine);
//   block → 16 warps, each a contiguous run of 256-element tiles ("part");
//   warp  → lane l of a tile reads elements [8l, 8l+8): one 16-byte load of bf16 per stream.
// Each thread keeps an online-softmax partial; lanes merge by a shuffle butterfly, parts merge
// in index order. Sampling needs the cumulative mass in index order: the part containing
// u·Z is found from the parts' masses, then that one part (a few KB, an L2 hit) is re-read and
// scanned in element order.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace nrl {

struct FwdParams {
    const void* logits;
    const void* ref;
    const uint8_t* allow;
    const float* add;
    const float* uniforms;
    int32_t* tokens;
    float* logp;
    float* ref_logp;
    float* kl;
    float* entropy;
    float* rowstats;
    uint8_t* status;
    float* parts;  // scratch [rows, nsplit·16, kPartFloats], used when nsplit > 1
    uint64_t rows;
    uint64_t allow_stride;
    uint64_t add_stride;
    uint32_t V;
    uint32_t nsplit;
    uint32_t tiles_per_block;  // tiles of 256 elements per block
    uint32_t parts_per_block;  // parts a block's range is cut into (kWarps, except in the grouped kernel)
    uint32_t flags;
    float tau;
};

// elements [begin, end) of part q (block split q / 16, warp q % 16)
__device__ __forceinline__ void part_range(const FwdParams& p, uint32_t q, uint32_t& begin, uint32_t& end) {
    uint32_t split = q / p.parts_per_block, w = q % p.parts_per_block;
    uint32_t tpw = (p.tiles_per_block + p.parts_per_block - 1) / p.parts_per_block;
    uint64_t t0 = (uint64_t)split * p.tiles_per_block + (uint64_t)w * tpw;
    uint64_t t1 = t0 + tpw;
    uint64_t tb = (uint64_t)(split + 1) * p.tiles_per_block;
    if (t1 > tb) t1 = tb;
    if (t0 > tb) t0 = tb;
    uint64_t b = t0 * kTile, e = t1 * kTile;
    begin = b > p.V ? p.V : (uint32_t)b;
    end = e > p.V ? p.V : (uint32_t)e;
}

// One 8-element vector of a row: the tempered, masked logits z (and zr).
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
struct VecLoader {
    Raw<DT> x, r;
    RawMask k;
    Raw<NRL_F32> am;
    __device__ __forceinline__ void load(const FwdParams& p, uint64_t row, uint32_t v, uint32_t end) {
        uint64_t e = row * p.V + v;
        if (VEC) {
            x.load(p.logits, e);
            if (REF) r.load(p.ref, e);
            if (ALLOW) k.load(p.allow + row * p.allow_stride, v);
            if (GENERAL && p.add) am.load(p.add, row * p.add_stride + v);
        } else {
            int n = (int)(end - v < (uint32_t)kVec ? end - v : (uint32_t)kVec);
            x.load_scalar(p.logits, e, n);
            if (REF) r.load_scalar(p.ref, e, n);
            if (ALLOW) k.load_scalar(p.allow + row * p.allow_stride, v, n);
            if (GENERAL && p.add) am.load_scalar(p.add, row * p.add_stride + v, n);
        }
    }
    __device__ __forceinline__ void values(const FwdParams& p, float z[8], float zr[8]) const {
        x.unpack(z);
        if (REF) r.unpack(zr);
        if (GENERAL) {
            // tempered_logits: logits / τ (skipped at τ = 1), then + additive mask
            if (p.tau != 1.0f) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    z[i] = __fdiv_rn(z[i], p.tau);
                    if (REF) zr[i] = __fdiv_rn(zr[i], p.tau);
                }
            }
            if (p.add) {
                float a[8];
                am.unpack(a);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    // an out-of-range lane of the scalar path carries −inf here, which leaves z at −inf
                    z[i] = z[i] + a[i];
                    if (REF) zr[i] = zr[i] + a[i];
                }
            }
        }
        if (ALLOW) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                // an excluded token becomes −FLT_MAX, not −inf: exp underflows to exactly 0 either
                // way, and no 0·inf or inf − inf can appear downstream
                bool ok = k.allowed(i);
                z[i] = ok ? z[i] : -FLT_MAX;
                if (REF) zr[i] = ok ? zr[i] : -FLT_MAX;
            }
        }
    }
};

__device__ __forceinline__ float fmin3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float warp_max_nan(float x) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) x = fmax_nan(x, __shfl_xor_sync(0xffffffffu, x, s));
    return x;
}

// A lane's running partial while it streams: the sums live as packed pairs (even elements in
// the low half, odd in the high half) so that the per-vector work is packed arithmetic only;
// the halves are added when the lane's partial is handed to the reduction tree.
struct Acc {
    f32x2 S2, W2, D2, Sr2;
    float m, mr;  // warp-wide maxima: the same in every lane of a warp
    float G;      // this lane's mass in the current chunk of the sampling log, at maximum m
};

__device__ __forceinline__ Acc acc_empty() {
    Acc a;
    a.S2 = a.W2 = a.D2 = a.Sr2 = pack2(0.f, 0.f);
    a.m = a.mr = NRL_NEG_INF;
    a.G = 0.f;
    return a;
}

__device__ __forceinline__ Partial acc_to_partial(const Acc& a) {
    Partial p;
    float x0, x1;
    unpack2(a.S2, x0, x1);
    p.S = x0 + x1;
    unpack2(a.W2, x0, x1);
    p.W = x0 + x1;
    unpack2(a.D2, x0, x1);
    p.D = x0 + x1;
    unpack2(a.Sr2, x0, x1);
    p.Sr = x0 + x1;
    p.m = a.m;
    p.mr = a.mr;
    return p;
}

// move the policy sums to a larger (or NaN) maximum mn
__device__ __forceinline__ void acc_rebase(Acc& a, float mn) {
    if (a.m != mn) {
        if (a.m == NRL_NEG_INF) {
            a.S2 = a.W2 = a.D2 = pack2(0.f, 0.f);
            a.G = 0.f;
        } else {
            const float dm = a.m - mn;
            const float c = expf(dm);  // accurate: a warp's maximum grows only ~ln(n) times per row
            const f32x2 c2 = pack2(c, c);
            a.W2 = mul2(fma2(a.S2, pack2(dm, dm), a.W2), c2);
            a.S2 = mul2(a.S2, c2);
            a.D2 = mul2(a.D2, c2);
            a.G *= c;
        }
        a.m = mn;
    }
}
__device__ __forceinline__ void acc_rebase_ref(Acc& a, float mn) {
    if (a.mr != mn) {
        if (a.mr == NRL_NEG_INF) {
            a.Sr2 = pack2(0.f, 0.f);
        } else {
            const float c = expf(a.mr - mn);
            a.Sr2 = mul2(a.Sr2, pack2(c, c));
        }
        a.mr = mn;
    }
}

// Fold one vector per lane into the lanes' partials. Called by all 32 lanes of a warp together
// (a lane without work passes −FLT_MAX everywhere). Values are finite or −FLT_MAX (excluded);
// real −inf logits are rare and are made safe in the slow block below.
//
// The running maxima are warp-wide: when some lane's vector exceeds the current maximum, every
// lane moves to the warp's new maximum at once. A warp's maximum grows only ~ln(n) times over a
// row, so one vote per vector keeps the rebase (an accurate expf), the −inf handling and the
// first-data case off the common path; with per-lane maxima a warp would take that path at
// almost every step. The common path is packed f32x2 arithmetic and 3-input min/max.
template <int N>
__device__ __forceinline__ float vec_max_nan(const float* z) {
    float m = fmax3_nan(fmax3_nan(fmax3_nan(z[0], z[1], z[2]), z[3], z[4]), fmax3_nan(z[5], z[6], z[7]), z[0]);
    if constexpr (N == 16) m = fmax3_nan(m, fmax3_nan(fmax3_nan(z[8], z[9], z[10]), z[11], z[12]), fmax3_nan(z[13], z[14], z[15]));
    return m;
}
template <int N>
__device__ __forceinline__ float vec_min(const float* z) {
    float m = fmin3(fmin3(fmin3(z[0], z[1], z[2]), z[3], z[4]), fmin3(z[5], z[6], z[7]), z[0]);
    if constexpr (N == 16) m = fmin3(m, fmin3(fmin3(z[8], z[9], z[10]), z[11], z[12]), fmin3(z[13], z[14], z[15]));
    return m;
}

// N = 8: one vector per lane. N = 16: the lane's vectors of two consecutive tiles folded as one step (one vote, one
// bookkeeping step for both).
template <bool REF, bool LOG, int N = 8>
__device__ __forceinline__ void accumulate(Acc& a, float* z, float* zr) {
    static_assert(N == 8 || N == 16, "one or two vectors");
    float vmax = vec_max_nan<N>(z);
    const float vmin = vec_min<N>(z);
    float rmax = NRL_NEG_INF;
    if (REF) rmax = vec_max_nan<N>(zr);
    const bool slow = !(vmax <= a.m) || vmin == NRL_NEG_INF || (REF && !(rmax <= a.mr));
    if (__any_sync(0xffffffffu, slow)) {
        if (vmin == NRL_NEG_INF) {
            // −inf logits: make them finite (exp underflows to exactly 0 either way) and keep
            // 0·inf and inf − inf out of the entropy and KL sums. The reference's entry is only
            // touched where the policy's was −inf, so a token the policy can draw but the
            // reference excludes still gives KL = +inf.
#pragma unroll
            for (int i = 0; i < N; i++) {
                if (z[i] == NRL_NEG_INF) {
                    z[i] = -FLT_MAX;
                    if (REF) zr[i] = fmaxf(zr[i], -FLT_MAX);
                }
            }
            vmax = fmax_nan(vmax, -FLT_MAX);
        }
        const float wm = warp_max_nan(vmax);
        if (!(wm <= -FLT_MAX)) acc_rebase(a, fmax_nan(a.m, wm));
        if (REF) {
            const float wr = warp_max_nan(rmax);
            if (wr != NRL_NEG_INF && !(wr <= -FLT_MAX)) acc_rebase_ref(a, fmax_nan(a.mr, wr));
        }
    }
    const f32x2 l2e = pack2(kLog2e, kLog2e);
    if (!(vmax <= -FLT_MAX)) {  // something allowed here (or a NaN)
        const f32x2 m2 = pack2(a.m, a.m);
        const f32x2 before = a.S2;
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const f32x2 zz = pack2(z[i], z[i + 1]);
            const f32x2 t = sub2(zz, m2);
            float a0, a1;
            unpack2(mul2(t, l2e), a0, a1);
            const f32x2 e = pack2(ex2_approx(a0), ex2_approx(a1));
            a.S2 = add2(a.S2, e);
            a.W2 = fma2(e, t, a.W2);
            if (REF) a.D2 = fma2(e, sub2(zz, pack2(zr[i], zr[i + 1])), a.D2);
        }
        if (LOG) {  // what this vector added to the lane's mass, for the sampling log
            float d0, d1;
            unpack2(sub2(a.S2, before), d0, d1);
            a.G += d0 + d1;
        }
    }
    if (REF) {
        if (rmax != NRL_NEG_INF && !(rmax <= -FLT_MAX)) {
            // (zr − mr) first, then the scale: folding mr·log2e into one fma would shift every
            // term of the row by the rounding of that product, and ln Zr with it
            const f32x2 mr2 = pack2(a.mr, a.mr);
#pragma unroll
            for (int i = 0; i < N; i += 2) {
                float a0, a1;
                unpack2(mul2(sub2(pack2(zr[i], zr[i + 1]), mr2), l2e), a0, a1);
                a.Sr2 = add2(a.Sr2, pack2(ex2_approx(a0), ex2_approx(a1)));
            }
        }
    }
}

// A thread block streams its range of one row and leaves 16 part partials in `sp`.
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__device__ __forceinline__ void stream_block(const FwdParams& p, uint64_t row, uint32_t split, Partial* sp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t begin, end;
    part_range(p, split * kWarps + warp, begin, end);
    Acc acc = acc_empty();
    // Software pipeline: kDepth tiles of this lane's loads are in flight while one is reduced
    // (about 64 KB per SM with two resident blocks: what HBM latency × bandwidth asks for).
#ifdef NRL_DEPTH
    constexpr int kDepth = NRL_DEPTH;
#else
    constexpr int kDepth = (REF || ALLOW || GENERAL || DT == NRL_F32) ? 3 : 4;
#endif
    VecLoader<DT, REF, ALLOW, GENERAL, VEC> buf[kDepth];
    uint32_t v = begin + lane * kVec;
#pragma unroll
    for (int d = 0; d < kDepth; d++)
        if (v + d * kTile < end) buf[d].load(p, row, v + d * kTile, end);
    for (uint32_t t0 = begin; t0 < end;) {  // t0: warp-uniform tile base
#pragma unroll
        for (int d = 0; d < kDepth; d++) {
            if (t0 < end) {
                float z[8], zr[8];
                if (v < end) {
                    buf[d].values(p, z, zr);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) z[i] = zr[i] = -FLT_MAX;
                }
                accumulate<REF, false>(acc, z, zr);
                uint32_t vn = v + kDepth * kTile;
                if (vn < end) buf[d].load(p, row, vn, end);
            }
            v += kTile;
            t0 += kTile;
        }
    }
    const Partial part = partial_warp_reduce(acc_to_partial(acc));
    if (lane == 0) sp[warp] = part;
}

// The unmasked fast path: each warp streams its part through a 4 KB ring in shared memory filled
// by asynchronous 16-byte copies (cp.async). A lane only ever reads back the bytes it copied
// itself, so its own wait_group is the only synchronisation. The ring keeps 4 KB per warp —
// 128 KB per SM with four resident blocks — in flight without holding registers, which is what
// lets the loads run far enough ahead of the arithmetic.
constexpr int kRingRows = 8;  // rows of 32 lanes × 16 B per warp

// The sampling log (shared memory, fused kernel only). While a warp streams its part it records,
// per chunk of the part and per lane, the mass the lane added in that chunk (relative to the
// warp's maximum at the chunk's end, also recorded). After the row's total is known, the chunk
// that holds u·Z is found from these numbers and only that chunk is read again — by one warp —
// instead of the whole part by the whole block. A chunk is a run of `tiles_per_chunk` tiles on
// the unmasked path (entries unused) or one batch of 32 queued vectors on the masked path
// (`entry` holds each lane's vector). A part that outgrows the log marks it overflowed and the
// block falls back to re-reading the whole part.
constexpr uint32_t kLogOverflow = 0xffffffffu;
constexpr uint32_t kNoEntry = 0xffffffffu;

template <int N, bool ENTRIES>
struct SampleLog {
    float mass[kWarps][N][32];
    uint32_t entry[ENTRIES ? kWarps : 1][ENTRIES ? N : 1][32];
    float cmax[kWarps][N];
    uint32_t count[kWarps];
    uint32_t tiles_per_chunk[kWarps];
};
constexpr int kLogDense = 64 / kWarps;     // chunks per part, unmasked path
#ifdef NRL_LOG_COMPACT
constexpr int kLogCompact = NRL_LOG_COMPACT;
#else
constexpr int kLogCompact = 128 / kWarps;  // batches per part, masked path
#endif
typedef SampleLog<kLogDense, false> DenseLog;
typedef SampleLog<kLogCompact, true> CompactLog;

// Streams part `part_index` of an unmasked row with one warp through `wring`, the calling warp's
// ring of kRingRows × 32 16-byte slots. With LOG, `sink(chunk, acc)` is called by all 32 lanes at
// the end of every chunk of `tiles_per_chunk` tiles (acc.G is the lane's mass in the chunk at
// maximum acc.m). Returns the part's partial (valid in lane 0).
template <int DT, bool REF, bool LOG, class Sink>
__device__ __forceinline__ Partial stream_part_async(const FwdParams& p, uint64_t row, uint32_t part_index, uint4* wring, Sink&& sink, uint32_t& chunks, uint32_t& tiles_per_chunk) {
    const int lane = threadIdx.x & 31;
    // 2-byte elements: a step takes several consecutive tiles, so that one wait and one round of ring and pointer
    // bookkeeping serve them all (the loop is bound by instruction issue, not by memory). Without a reference stream
    // four tiles, folded 16 elements at a time (one vote per two vectors): +26 % over one tile per step. With one, two
    // tiles folded 8 + 8: 32 values at once do not fit 64 registers (the 16-wide fold spilled and gained nothing), and
    // four tiles of two streams would leave the 4 KB ring a single slot: +6 %.
    // 4-byte elements without a reference stream: two tiles, one 16-wide fold (+3 %).
    constexpr int kT = DT == NRL_BF16 ? (REF ? 2 : 4) : (REF ? 1 : 2);  // tiles per step
    constexpr bool kWide = kT >= 2 && !REF;
    constexpr int kPer = (DT == NRL_F32 ? 2 : 1);     // 16-byte pieces per lane per stream per tile
    constexpr int kRows = kPer * (REF ? 2 : 1) * kT;  // ring rows one step takes
    constexpr int kSlots = kRingRows / kRows;         // steps in flight
    constexpr uint32_t kEsize = (DT == NRL_F32 ? 4 : 2);
    constexpr uint32_t kStep = kT * kTile;            // elements per step
    uint32_t begin, end;
    part_range(p, part_index, begin, end);
    Acc acc = acc_empty();
    const uint32_t base = smem_addr(wring + lane);  // this lane's column of the ring
    // Every warp-wide copy covers 512 contiguous bytes. With 2-byte elements a lane's piece is its
    // 8 elements of the tile; with 4-byte elements a lane takes two pieces of 4 elements, 128
    // elements apart (lane·4 … and 128 + lane·4 …), so that neither copy touches half sectors.
    constexpr uint32_t kLaneElems = 16 / kEsize;  // elements per 16-byte piece
    constexpr uint32_t kPieceGap = DT == NRL_F32 ? 128 : kTile;  // elements between a lane's two pieces: the next tile (bf16 pairs) or half a tile (f32)
    constexpr int kPieces = kPer * kT;                     // pieces per lane per stream per step
    const char* xp = (const char*)p.logits + (row * p.V + begin + lane * kLaneElems) * kEsize;
    const char* rp = REF ? (const char*)p.ref + (row * p.V + begin + lane * kLaneElems) * kEsize : nullptr;
    uint32_t v = begin + lane * kLaneElems;  // this lane's first element of the step it consumes next
    // sampling log: chunks of `gsz` tiles (a whole number of steps), at most kLogDense of them
    const uint32_t ntiles = (end - begin + kTile - 1) / kTile;
    const uint32_t gsz = ((ntiles + kLogDense - 1) / kLogDense + kT - 1) / kT * kT;
    uint32_t left = gsz, chunk = 0;
    auto flush = [&]() {
        sink(chunk, acc);
        acc.G = 0.f;
        chunk++;
        left = gsz;
    };
    auto issue = [&](int slot, uint32_t vv, const char* xq, const char* rq) {
#pragma unroll
        for (int k = 0; k < kPieces; k++) {
            if (vv + k * kPieceGap < end) {
                cp_async16(base + (slot * kRows + k) * 512, xq + kPieceGap * kEsize * k);
                if (REF) cp_async16(base + (slot * kRows + kPieces + k) * 512, rq + kPieceGap * kEsize * k);
            }
        }
        cp_async_commit();  // one group per step, empty or not, so that the group count stays in step
    };
#pragma unroll
    for (int s = 0; s < kSlots; s++) issue(s, v + s * kStep, xp + (size_t)s * kStep * kEsize, REF ? rp + (size_t)s * kStep * kEsize : nullptr);
    for (uint32_t t0 = begin; t0 < end; t0 += kSlots * kStep) {  // warp-uniform
        // not unrolled: one copy of the per-step arithmetic keeps the loop inside the instruction cache
        // (measured 4 % faster with a reference stream, 8 % without, than the loop unrolled over the slots)
#pragma unroll 1
        for (int s = 0; s < kSlots; s++) {
            cp_async_wait<kSlots - 1>();  // the oldest step has landed
            if (t0 + s * kStep < end) {  // warp-uniform: the step exists
                if constexpr (DT == NRL_F32) {
                    // four floats per piece; without a reference stream a step is two tiles, folded 16 at a time
                    float z[8 * kT], zr[8 * kT];
#pragma unroll
                    for (int k = 0; k < kPieces; k++) {
                        const uint4 q = lds16(base + (s * kRows + k) * 512);
                        z[4 * k] = __uint_as_float(q.x); z[4 * k + 1] = __uint_as_float(q.y); z[4 * k + 2] = __uint_as_float(q.z); z[4 * k + 3] = __uint_as_float(q.w);
                        if (REF) {
                            const uint4 r = lds16(base + (s * kRows + kPieces + k) * 512);
                            zr[4 * k] = __uint_as_float(r.x); zr[4 * k + 1] = __uint_as_float(r.y); zr[4 * k + 2] = __uint_as_float(r.z); zr[4 * k + 3] = __uint_as_float(r.w);
                        }
                        // a piece past the end of a ragged last tile: nothing was copied, nothing to add
                        if (v + k * kPieceGap >= end) {
#pragma unroll
                            for (int i = 4 * k; i < 4 * k + 4; i++) z[i] = zr[i] = -FLT_MAX;
                        }
                    }
                    accumulate<REF, LOG, 8 * kT>(acc, z, zr);
                } else if constexpr (kWide) {
#pragma unroll
                    for (int h = 0; h < kT / 2; h++) {
                        float z[16], zr[16];
#pragma unroll
                        for (int k = 0; k < 2; k++) {
                            Raw<DT> x;
                            x.q = lds16(base + (s * kRows + 2 * h + k) * 512);
                            x.unpack(z + 8 * k);
                            if (v + (2 * h + k) * kTile >= end) {
#pragma unroll
                                for (int i = 8 * k; i < 8 * k + 8; i++) z[i] = -FLT_MAX;
                            }
                        }
                        accumulate<false, LOG, 16>(acc, z, zr);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < kT; k++) {
                        float z[8], zr[8];
                        Raw<DT> x, r;
                        x.q = lds16(base + (s * kRows + k) * 512);
                        x.unpack(z);
                        if (REF) {
                            r.q = lds16(base + (s * kRows + kT + k) * 512);
                            r.unpack(zr);
                        }
                        if (v + k * kTile >= end) {
#pragma unroll
                            for (int i = 0; i < 8; i++) z[i] = zr[i] = -FLT_MAX;
                        }
                        accumulate<REF, LOG>(acc, z, zr);
                    }
                }
                if (LOG) {
                    left -= kT;
                    if (left == 0) flush();
                }
            }
            // refill the slot just consumed with the step kSlots ahead
            issue(s, v + kSlots * kStep, xp + (size_t)kSlots * kStep * kEsize, REF ? rp + (size_t)kSlots * kStep * kEsize : nullptr);
            v += kStep;
            xp += (size_t)kStep * kEsize;
            if (REF) rp += (size_t)kStep * kEsize;
        }
    }
    cp_async_wait<0>();
    if (LOG && left != gsz) flush();
    chunks = chunk;
    tiles_per_chunk = gsz;
    return partial_warp_reduce(acc_to_partial(acc));
}

// One block streams its range of an unmasked row: warp w takes part split·kWarps + w and logs per lane.
template <int DT, bool REF, bool LOG>
__device__ __forceinline__ void stream_block_async(const FwdParams& p, uint64_t row, uint32_t split, Partial* sp, uint4* ring, DenseLog* log) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t chunks = 0, per = 0;
    const Partial part = stream_part_async<DT, REF, LOG>(p, row, split * kWarps + warp, ring + warp * (kRingRows * 32), [&](uint32_t chunk, const Acc& acc) {
        log->mass[warp][chunk][lane] = acc.G;
        if (lane == 0) log->cmax[warp][chunk] = acc.m;
    }, chunks, per);
    if (LOG && lane == 0) {
        log->count[warp] = chunks;
        log->tiles_per_chunk[warp] = per;
    }
    if (lane == 0) sp[warp] = part;
}

// The same for rows with a byte allow-mask, when most of the vocabulary is excluded (grammar
// masks allow a few per cent of it): an excluded logit cannot affect any output, so it is not
// read. Each warp scans its part's mask bytes tile by tile (1 byte per element, coalesced) and
// queues the 8-element vectors that hold at least one allowed token in a 64-entry ring in shared
// memory; whenever 32 are queued, every lane takes one, loads its logits / reference / mask
// bytes and folds it into its partial. Issued arithmetic therefore runs on 32 busy lanes instead
// of the one or two per tile that have work, and HBM traffic drops to the mask plus the 32-byte
// sectors that contain an allowed token. The batch order depends only on the mask, so results
// stay bitwise reproducible.
constexpr int kQueue = 256;  // ring entries per warp: 31 left over + 4 tiles × 32 lanes, rounded up
constexpr int kAhead = 4;    // mask tiles scanned per group
#ifndef NRL_AHEAD_REF
#define NRL_AHEAD_REF 4
#endif
constexpr int kAheadRef = NRL_AHEAD_REF;  // the same with a reference stream (more registers held per vector)

// Streams part `part_index` of a row with one warp. `wq` is the calling warp's kQueue-entry ring;
// `sink(batch, acc, pend_v)` is called by all 32 lanes once per folded batch when LOG (acc.G is
// the lane's mass in that batch at maximum acc.m, pend_v the vector the lane folded or kNoEntry)
// and must leave acc.G alone. Returns the part's partial (valid in lane 0) and, in `batches`, the
// number of batches folded.
template <int DT, bool REF, bool LOG, class Sink>
__device__ __forceinline__ Partial stream_part_compact(const FwdParams& p, uint64_t row, uint32_t part_index, uint32_t* wq, Sink&& sink, uint32_t& batches) {
    constexpr int kA = REF ? kAheadRef : kAhead;  // mask tiles scanned per group
    const int lane = threadIdx.x & 31;
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t begin, end;
    part_range(p, part_index, begin, end);
    typedef VecLoader<DT, REF, true, false, true> Loader;
    Acc acc = acc_empty();
    Loader pend;
    bool pend_ok = false, pend_any = false;
    uint32_t pend_v = kNoEntry, batch = 0;  // the vector this lane holds in `pend`; batches folded so far
    uint32_t head = 0, count = 0;  // warp-uniform ring state

    // this lane's mask bytes of the tile at `v`: pointer arithmetic is one 64-bit add per group
    // (with a bit per token, kMaskStep bytes of the row's mask cover one element step of 8)
#if NRL_MASK_BITS
    const uint8_t* mp = p.allow + row * p.allow_stride + ((begin + lane * kVec) >> 3);
    constexpr uint32_t kTileMask = kTile / 8;  // mask bytes a tile spans
#else
    const uint8_t* mp = p.allow + row * p.allow_stride + begin + lane * kVec;
    constexpr uint32_t kTileMask = kTile;
#endif
    uint32_t v = begin + lane * kVec;
    uint32_t t0 = begin;  // warp-uniform tile base of the group in mk[]
    uint32_t mk[kA];  // non-zero iff the tile's vector of this lane allows a token: all the scan needs
    MaskAny mn[kA];
#pragma unroll
    for (int j = 0; j < kA; j++) {
        const MaskAny q = (v + j * kTile < end) ? ldg_mask_any(mp + j * kTileMask, 0) : mask_any_none();
        mk[j] = mask_any_value(q);
    }
    // One loop with one copy of the arithmetic (a small instruction footprint): each turn scans
    // a group of mask tiles if any is left, then folds batches while at least 32 vectors are
    // queued; after the last group it drains the queue and the pending batch.
    for (;;) {
        const bool scanning = t0 < end;
        if (scanning) {
            // the next group's mask bytes fly while this group is scanned, and the group eight
            // ahead is pulled into L2 (one 128-byte line per lane 0..7) so that its loads are
            // short when their turn comes
            const uint8_t* np = mp + kA * kTileMask;
            const uint32_t nv = v + kA * kTile;
#if !NRL_MASK_BITS
            if (lane < 8 && t0 + 8 * kA * kTile + lane * 128 < end) prefetch_l2(mp - lane * kVec + 8 * kA * kTile + lane * 128);
#endif
#pragma unroll
            for (int j = 0; j < kA; j++) mn[j] = (nv + j * kTile < end) ? ldg_mask_any(np + j * kTileMask, 0) : mask_any_none();
#pragma unroll
            for (int j = 0; j < kA; j++) {
                const bool nz = mk[j] != 0u;
                const uint32_t ball = __ballot_sync(0xffffffffu, nz);
                if (nz) wq[(head + count + __popc(ball & lt)) & (kQueue - 1)] = v + j * kTile;
                count += __popc(ball);
            }
#pragma unroll
            for (int j = 0; j < kA; j++) mk[j] = mask_any_value(mn[j]);
            mp = np;
            v = nv;
            t0 += kA * kTile;
            __syncwarp();
        }
        while (count >= 32 || (!scanning && (count > 0 || pend_any))) {
            // lane l takes queue entry l; the previous batch is folded while these loads fly
            const uint32_t n = count < 32 ? count : 32;
            Loader nxt;
            const bool ok = (uint32_t)lane < n;
            const uint32_t nv_entry = ok ? wq[(head + lane) & (kQueue - 1)] : kNoEntry;
            if (ok) nxt.load(p, row, nv_entry, end);
            head = (head + n) & (kQueue - 1);
            count -= n;
            if (pend_any) {  // warp-uniform; lanes without an entry fold an empty vector
                float z[8], zr[8];
                if (pend_ok) {
                    pend.values(p, z, zr);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) z[i] = zr[i] = -FLT_MAX;
                }
                accumulate<REF, LOG>(acc, z, zr);
                if (LOG) {  // one log chunk per batch: the lane's vector and what it added
                    sink(batch, acc, pend_v);
                    acc.G = 0.f;
                    batch++;
                }
            }
            pend = nxt;
            pend_v = nv_entry;
            pend_ok = ok;
            pend_any = n > 0;
        }
        if (!scanning) break;
        __syncwarp();  // the batch's entries are read before the next group's pushes can reuse slots
    }
    batches = batch;
    return partial_warp_reduce(acc_to_partial(acc));
}

// One block streams its range of a row: warp w takes part split·kWarps + w and logs per lane.
template <int DT, bool REF, bool LOG>
__device__ __forceinline__ void stream_block_compact(const FwdParams& p, uint64_t row, uint32_t split, Partial* sp, uint32_t* queue, CompactLog* log) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t batches = 0;
    const Partial part = stream_part_compact<DT, REF, LOG>(p, row, split * kWarps + warp, queue + warp * kQueue, [&](uint32_t batch, const Acc& acc, uint32_t pend_v) {
        if (batch < (uint32_t)kLogCompact) {
            log->mass[warp][batch][lane] = acc.G;
            log->entry[warp][batch][lane] = pend_v;
            if (lane == 0) log->cmax[warp][batch] = acc.m;
        }
    }, batches);
    if (LOG && lane == 0) log->count[warp] = batches <= (uint32_t)kLogCompact ? batches : kLogOverflow;
    if (lane == 0) sp[warp] = part;
}

struct RowResult {
    double Z, Zr, W, D;  // totals at the row maxima
    float m, mr;
    float lnZ, lnZr, kl, ent;
    uint32_t status;
    uint32_t part;       // the part holding the token (sampling / greedy)
    double resid;        // u·Z minus the mass before that part
};

// Warp 0 merges `nparts` partials (index order) into the row's result and, for sampling,
// finds the part containing u·Z. get(q) returns partial q.
template <class Get>
__device__ __forceinline__ void finalize_row(const FwdParams& p, uint64_t row, uint32_t nparts, Get get, RowResult* out) {
    const int lane = threadIdx.x & 31;
    const uint32_t per = (nparts + 31) / 32;  // parts per lane, contiguous
    // pass 1: the row maxima
    float m = NRL_NEG_INF, mr = NRL_NEG_INF;
    for (uint32_t i = 0; i < per; i++) {
        uint32_t q = lane * per + i;
        if (q < nparts) {
            Partial a = get(q);
            m = fmax_nan(m, a.m);
            mr = fmax_nan(mr, a.mr);
        }
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        m = fmax_nan(m, __shfl_xor_sync(0xffffffffu, m, s));
        mr = fmax_nan(mr, __shfl_xor_sync(0xffffffffu, mr, s));
    }
    // pass 2: masses at the row maxima, in f64, summed in index order
    double S = 0.0, W = 0.0, D = 0.0, Sr = 0.0;
    for (uint32_t i = 0; i < per; i++) {
        uint32_t q = lane * per + i;
        if (q < nparts) {
            Partial a = get(q);
            if (a.m != NRL_NEG_INF && a.S > 0.f) {
                // f32 expf (1 ulp) is enough for the rescale: its error enters the row's mass
                // weighted by e^dm·|dm|, at most a few 1e-8, and it is ~10× cheaper than f64 exp
                double dm = (double)a.m - (double)m;
                double c = (double)expf(a.m - m);
                S += c * (double)a.S;
                W += c * ((double)a.W + (double)a.S * dm);
                D += c * (double)a.D;
            }
            if (a.mr != NRL_NEG_INF) Sr += (double)expf(a.mr - mr) * (double)a.Sr;
        }
    }
    double Sin = warp_scan_incl(S, lane);
    double Z = __shfl_sync(0xffffffffu, Sin, 31);
    double Wt = warp_scan_incl(W, lane), Dt = warp_scan_incl(D, lane), Srt = warp_scan_incl(Sr, lane);
    Wt = __shfl_sync(0xffffffffu, Wt, 31);
    Dt = __shfl_sync(0xffffffffu, Dt, 31);
    Srt = __shfl_sync(0xffffffffu, Srt, 31);

    uint32_t status = 0;
    if (m != m) status |= 2u;
    else if (m == NRL_NEG_INF) status |= 1u;

    uint32_t part = 0;
    double resid = 0.0;
    if (!status && (p.flags & NRL_FWD_SAMPLE)) {
        double t = (double)p.uniforms[row] * Z;
        double Sex = Sin - S;  // mass before this lane's parts
        bool mine = Sin > t;   // the first lane whose inclusive mass exceeds t holds the token
        uint32_t ball = __ballot_sync(0xffffffffu, mine);
        uint32_t has = __ballot_sync(0xffffffffu, S > 0.0);
        int owner = ball ? (__ffs(ball) - 1) : (31 - __clz(has));  // rounding only: last lane with mass
        uint32_t my_part = 0;
        double my_res = 0.0;
        if (lane == owner) {
            double c = Sex;
            uint32_t last = lane * per;
            bool found = false;
            for (uint32_t i = 0; i < per && !found; i++) {
                uint32_t q = lane * per + i;
                if (q >= nparts) break;
                Partial a = get(q);
                if (!(a.m != NRL_NEG_INF && a.S > 0.f)) continue;
                double mass = (double)expf(a.m - m) * (double)a.S;
                last = q;
                if (c + mass > t) {
                    my_part = q;
                    my_res = t - c;
                    found = true;
                } else {
                    c += mass;
                }
            }
            if (!found) {
                my_part = last;
                my_res = 1e300;  // past the end: the scan below takes the part's last token with mass
            }
        }
        part = __shfl_sync(0xffffffffu, my_part, owner);
        resid = __shfl_sync(0xffffffffu, my_res, owner);
    } else if (!status && (p.flags & NRL_FWD_GREEDY)) {
        // the first part whose maximum is the row's
        uint32_t first = 0xffffffffu;
        for (uint32_t i = 0; i < per; i++) {
            uint32_t q = lane * per + i;
            if (q < nparts && first == 0xffffffffu && get(q).m == m) first = q;
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            uint32_t o = __shfl_xor_sync(0xffffffffu, first, s);
            first = o < first ? o : first;
        }
        part = first;
    }
    // both logarithms at once: lane 1 takes the reference's, the others the policy's
    const double lg = log(lane == 1 ? Srt : Z);
    const double lnZ = __shfl_sync(0xffffffffu, lg, 0), lnZr = __shfl_sync(0xffffffffu, lg, 1);
    if (lane == 0) {
        RowResult r;
        r.Z = Z; r.Zr = Srt; r.W = Wt; r.D = Dt;
        r.m = m; r.mr = mr;
        r.lnZ = (float)lnZ;
        r.lnZr = (float)lnZr;
        r.ent = (float)(lnZ - Wt / Z);
        // KL = Σπ(z − zr) − (m + ln Z) + (mr + ln Zr)
        r.kl = (float)(Dt / Z - ((double)m - (double)mr) - (lnZ - lnZr));
        r.status = status;
        r.part = part;
        r.resid = resid;
        *out = r;
    }
}

}  // namespace nrl
