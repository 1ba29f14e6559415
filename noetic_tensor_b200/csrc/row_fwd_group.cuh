// The grouped row forward (many rows on the vectorised fast paths, sampling or given tokens).
//
// In the one-block-per-row kernel a row ends with a tail — merge the part partials, find the
// token, read its logits, write the outputs — during which one warp works through a chain of
// dependent loads while the block's other warps wait, and before it every warp waits for the
// row's slowest part. Here a block takes a group of consecutive rows (group_rows). Its warps take
// (row, part) tickets from a counter in shared memory, rows in order, and stream one part per
// ticket into the row's own result buffer, so heavy and light parts balance over the group and
// nothing is waited for. After one barrier at the end the rows' tails run side by side, one warp
// per row: their latency is paid once per group instead of once per row. There is no spin and
// nothing that could hang.
//
// Every result is a pure function of (row, part): which warp streams a part and when does not
// enter any sum, and parts are merged in index order, so results are bitwise reproducible and
// the row statistics equal the one-block-per-row kernel's bit for bit.
#pragma once
#include "row_fwd_kernels.cuh"

namespace nrl {

#ifndef NRL_GROUP_ROWS
#define NRL_GROUP_ROWS 4
#endif
#ifndef NRL_GROUP_SPLIT
#define NRL_GROUP_SPLIT 1
#endif
#ifndef NRL_GROUP_ROWS_DENSE
#define NRL_GROUP_ROWS_DENSE 4
#endif
// rows per block: the per-row buffers of masked rows hold the batch log and are larger
template <bool ALLOW>
__host__ __device__ constexpr int group_rows() {
    return ALLOW ? NRL_GROUP_ROWS : NRL_GROUP_ROWS_DENSE;
}
// Parts per row = kGroupSplit · kWarps. Finer parts would balance the tickets better (the warp
// that runs a row's tail falls behind and tends to take the next row's last ticket too), but each
// part pays for filling and draining the load pipeline: one part per warp measured fastest.
constexpr int kGroupSplit = NRL_GROUP_SPLIT;
constexpr int kGroupParts = kGroupSplit * kWarps;
#ifndef NRL_PLOG
#define NRL_PLOG (64 / kGroupSplit)
#endif
constexpr int kPLog = NRL_PLOG;                   // logged batches per part, masked rows

// What the streaming pass leaves per part for the token pick.
// Masked rows: a batch is 32 consecutive live vectors (vectors with an allowed token) of the part
// in index order; per batch the warp's mass at maximum cmax and the batch's first vector as its
// index within the part; the batch's other vectors are found again from the mask.
struct MaskedPartLog {
    float mass[kPLog];
    float cmax[kPLog];
    uint16_t first[kPLog];
    uint32_t count;  // batches folded, or kLogOverflow
};
// Unmasked rows: a chunk is `tiles` consecutive tiles of the part; per chunk the warp's mass at
// maximum cmax.
struct DensePartLog {
    float mass[kLogDense];
    float cmax[kLogDense];
    uint32_t count;
    uint32_t tiles;
};

// Lane l holds vector `vv` (or kNoEntry) of 32 vectors in index order; `run` is the mass before
// them. Returns the token at which the running mass first exceeds `target`, or −1 if the vectors
// end first (then `run` has them added and `last` is the lane's last token with mass, if any).
template <int DT, bool ALLOW>
__device__ __forceinline__ int32_t scan_batch(const FwdParams& p, uint64_t row, uint32_t vv, uint32_t end, float m, double& run, double target, int32_t& last) {
    typedef VecLoader<DT, false, ALLOW, false, true> Loader;
    const int lane = threadIdx.x & 31;
    float e[8];
    double s = 0.0;
    if (vv != kNoEntry) {
        Loader ld;
        ld.load(p, row, vv, end);
        float z[8], zr[8];
        ld.values(p, z, zr);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            e[i] = ex2_approx((fmaxf(z[i], -FLT_MAX) - m) * kLog2e);
            s += (double)e[i];
            if (e[i] > 0.f) last = (int32_t)(vv + i);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) e[i] = 0.f;
    }
    const double incl = warp_scan_incl(s, lane);
    const bool mine = s > 0.0 && run + incl > target;
    const uint32_t ball = __ballot_sync(0xffffffffu, mine);
    int32_t token = -1;
    if (ball) {
        const int owner = __ffs(ball) - 1;
        int32_t tok = -1;
        if (lane == owner) {
            double c = run + (incl - s);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                c += (double)e[i];
                if (tok < 0 && e[i] > 0.f && c > target) tok = (int32_t)(vv + i);
            }
            if (tok < 0) tok = last;  // rounding inside the vector
        }
        token = __shfl_sync(0xffffffffu, tok, owner);
    }
    run += __shfl_sync(0xffffffffu, incl, 31);
    return token;
}

__device__ __forceinline__ int32_t warp_max_i32(int32_t x) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        int32_t o = __shfl_xor_sync(0xffffffffu, x, s);
        x = o > x ? o : x;
    }
    return x;
}

// One warp: the first 32 live vectors of the part from element `v0` on, in index order, handed
// one per lane (kNoEntry past the last). `slots` is 32 words of this warp's own shared memory.
// Mask tiles are read four at a time; the loop ends at the part's end or with 32 vectors found.
__device__ __forceinline__ uint32_t regather_batch(const FwdParams& p, uint64_t row, uint32_t begin, uint32_t end, uint32_t v0, uint32_t* slots) {
    const int lane = threadIdx.x & 31;
    const uint32_t lt = (1u << lane) - 1u;
    const uint8_t* mrow = p.allow + row * p.allow_stride;
    uint32_t got = 0;
    __syncwarp();
    for (uint32_t t0 = begin + (v0 - begin) / kTile * kTile; t0 < end && got < 32; t0 += 4 * kTile) {
        uint2 q[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t v = t0 + j * kTile + lane * kVec;
            q[j] = (v >= v0 && v < end) ? ldg_mask8(mrow, v) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const bool live = (q[j].x | q[j].y) != 0u;
            const uint32_t ball = __ballot_sync(0xffffffffu, live);
            const uint32_t rank = got + __popc(ball & lt);
            if (live && rank < 32) slots[rank] = t0 + j * kTile + lane * kVec;
            got += __popc(ball);
        }
    }
    __syncwarp();
    return ((uint32_t)lane < got) ? slots[lane] : kNoEntry;
}

// The chunk (of up to 64, two per lane) that holds `resid`, from the chunks' masses x[0] (chunk
// `lane`) and x[1] (chunk `lane + 32`) at the row maximum: returns its index, the mass before it
// in `before`, and whether rounding left no crossing (`take_last`: the last chunk with mass is
// returned). −1 if no chunk has mass.
__device__ __forceinline__ int find_chunk(const double x[2], double resid, double& before, bool& take_last) {
    const int lane = threadIdx.x & 31;
    const double lo_incl = warp_scan_incl(x[0], lane);
    const double lo_total = __shfl_sync(0xffffffffu, lo_incl, 31);
    const double hi_incl = lo_total + warp_scan_incl(x[1], lane);
    const uint32_t cross_lo = __ballot_sync(0xffffffffu, x[0] > 0.0 && lo_incl > resid);
    const uint32_t cross_hi = __ballot_sync(0xffffffffu, x[1] > 0.0 && hi_incl > resid);
    const uint32_t has_lo = __ballot_sync(0xffffffffu, x[0] > 0.0);
    const uint32_t has_hi = __ballot_sync(0xffffffffu, x[1] > 0.0);
    if (!(has_lo | has_hi)) return -1;
    take_last = !(cross_lo | cross_hi);
    int c;
    if (take_last) c = has_hi ? 32 + (31 - __clz(has_hi)) : 31 - __clz(has_lo);
    else c = cross_lo ? __ffs(cross_lo) - 1 : 32 + __ffs(cross_hi) - 1;
    before = c < 32 ? __shfl_sync(0xffffffffu, lo_incl - x[0], c) : __shfl_sync(0xffffffffu, hi_incl - x[1], c - 32);
    return c;
}

template <class Log>
__device__ __forceinline__ void chunk_masses(const Log* log, uint32_t n, float m, double x[2]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t c = (uint32_t)lane + 32u * h;
        x[h] = 0.0;
        if (c < n) {
            const float cm = log->cmax[c];
            x[h] = cm == NRL_NEG_INF ? 0.0 : (double)log->mass[c] * (double)expf(cm - m);
        }
    }
}

// One warp: the token inside part `res.part` of a masked row from the part's log: the batch that
// holds res.resid is found from the logged masses, its vectors again from the mask, and read again.
template <int DT>
__device__ __forceinline__ int32_t pick_from_part_log(const FwdParams& p, uint64_t row, const RowResult& res, const MaskedPartLog* log, uint32_t* slots) {
    uint32_t begin, end;
    part_range(p, res.part, begin, end);
    double x[2], before = 0.0;
    bool take_last = false;
    chunk_masses(log, log->count, res.m, x);
    const int c = find_chunk(x, res.resid, before, take_last);
    if (c < 0) return -1;  // the part holds no mass at all
    const uint32_t v0 = begin + (uint32_t)log->first[c] * kVec;
    const uint32_t vv = regather_batch(p, row, begin, end, v0, slots);
    double run = 0.0;
    int32_t last = -1;
    int32_t tok = scan_batch<DT, true>(p, row, vv, end, res.m, run, take_last ? 1e300 : res.resid - before, last);
    if (tok < 0) tok = warp_max_i32(last);
    return tok;
}

// One warp, masked row, no log (a part that outgrew it): scan the part's vectors 32 at a time,
// mask bytes first, in index order.
template <int DT>
__device__ __forceinline__ int32_t pick_from_part_scan(const FwdParams& p, uint64_t row, const RowResult& res) {
    const int lane = threadIdx.x & 31;
    uint32_t begin, end;
    part_range(p, res.part, begin, end);
    const uint8_t* mrow = p.allow + row * p.allow_stride;
    double run = 0.0;
    int32_t last = -1;
    for (uint32_t t0 = begin; t0 < end; t0 += kTile) {
        const uint32_t v = t0 + lane * kVec;
        RawMask mk;
        mk.q = make_uint2(0u, 0u);
        if (v < end) mk.load(mrow, v);
        if (!__any_sync(0xffffffffu, mk.any())) continue;
        int32_t tok = scan_batch<DT, true>(p, row, mk.any() ? v : kNoEntry, end, res.m, run, res.resid, last);
        if (tok >= 0) return tok;
    }
    return warp_max_i32(last);
}

// One warp, unmasked row: the chunk that holds res.resid from the logged chunk masses, then that
// chunk's tiles in index order.
template <int DT>
__device__ __forceinline__ int32_t pick_from_chunk_log(const FwdParams& p, uint64_t row, const RowResult& res, const DensePartLog* log) {
    const int lane = threadIdx.x & 31;
    uint32_t begin, end;
    part_range(p, res.part, begin, end);
    double x[2], before = 0.0;
    bool take_last = false;
    chunk_masses(log, log->count, res.m, x);
    const int c = find_chunk(x, res.resid, before, take_last);
    if (c < 0) return -1;
    const uint32_t ca = begin + (uint32_t)c * log->tiles * kTile;
    uint32_t cb = ca + log->tiles * kTile;
    if (cb > end) cb = end;
    const double target = take_last ? 1e300 : res.resid - before;
    double run = 0.0;
    int32_t last = -1;
    for (uint32_t t0 = ca; t0 < cb; t0 += kTile) {
        const uint32_t v = t0 + lane * kVec;
        int32_t tok = scan_batch<DT, false>(p, row, v < cb ? v : kNoEntry, end, res.m, run, target, last);
        if (tok >= 0) return tok;
    }
    return warp_max_i32(last);
}

template <bool ALLOW>
struct GroupShared {
    typedef typename std::conditional<ALLOW, MaskedPartLog, DensePartLog>::type Log;
    Partial sp[group_rows<ALLOW>()][kGroupParts];
    Log log[group_rows<ALLOW>()][kGroupParts];
    RowResult res[kWarps];
    uint32_t next_ticket;
};

// Blocks per SM. With a reference stream the masked loop holds two more 16-byte loads per vector
// in flight: three blocks per SM (80 registers per thread) measured faster than four (64, with
// spills).
#ifndef NRL_GROUP_BLOCKS_REF
#define NRL_GROUP_BLOCKS_REF 3
#endif
#ifndef NRL_GROUP_BLOCKS_DENSE_REF
#define NRL_GROUP_BLOCKS_DENSE_REF 4
#endif
#ifndef NRL_GROUP_BLOCKS_NOREF
#define NRL_GROUP_BLOCKS_NOREF (1024 / kThreads)
#endif
template <bool REF, bool ALLOW>
constexpr int group_blocks() {
    return REF ? (ALLOW ? NRL_GROUP_BLOCKS_REF : NRL_GROUP_BLOCKS_DENSE_REF) : NRL_GROUP_BLOCKS_NOREF;
}

template <int DT, bool REF, bool ALLOW>
__global__ void __launch_bounds__(kThreads, group_blocks<REF, ALLOW>()) row_fwd_grouped(FwdParams p) {
    __shared__ GroupShared<ALLOW> sh;
    // the staging area of the streaming loop: the vector queue (masked) or the copy ring (unmasked)
    __shared__ __align__(16) uint32_t stage[ALLOW ? kWarps * kQueue : kWarps * kRingRows * 32 * 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) sh.next_ticket = 0u;
    __syncthreads();
    const uint64_t row0 = (uint64_t)blockIdx.x * group_rows<ALLOW>();
    const uint64_t left = p.rows - row0;
    const uint32_t nrows = (uint32_t)(left < (uint64_t)group_rows<ALLOW>() ? left : (uint64_t)group_rows<ALLOW>());
    const bool sampling = (p.flags & NRL_FWD_SAMPLE) != 0;
    uint32_t* wstage = stage + warp * (ALLOW ? kQueue : kRingRows * 32 * 4);

    // one part of one row of the group, streamed by the calling warp and delivered to the row's buffer
    auto stream_one = [&](uint32_t b, uint32_t part) {
        const uint64_t row = row0 + b;
        auto* lg = &sh.log[b][part];
        Partial mine;
        if constexpr (ALLOW) {
            uint32_t batches = 0, part_begin, part_end;
            part_range(p, part, part_begin, part_end);
            auto sink = [&](uint32_t batch, const Acc& acc, uint32_t pend_v) {
                float g = acc.G;
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) g += __shfl_xor_sync(0xffffffffu, g, s);
                if (lane == 0 && batch < (uint32_t)kPLog) {
                    lg->mass[batch] = g;
                    lg->cmax[batch] = acc.m;
                    lg->first[batch] = (uint16_t)((pend_v - part_begin) / kVec);  // lane 0 holds the batch's first vector
                }
            };
            if (sampling) mine = stream_part_compact<DT, REF, true>(p, row, part, wstage, sink, batches);
            else mine = stream_part_compact<DT, REF, false>(p, row, part, wstage, sink, batches);
            if (lane == 0) lg->count = batches <= (uint32_t)kPLog ? batches : kLogOverflow;
        } else {
            uint32_t chunks = 0, per = 0;
            auto sink = [&](uint32_t chunk, const Acc& acc) {
                float g = acc.G;
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) g += __shfl_xor_sync(0xffffffffu, g, s);
                if (lane == 0) {
                    lg->mass[chunk] = g;
                    lg->cmax[chunk] = acc.m;
                }
            };
            uint4* wring = reinterpret_cast<uint4*>(wstage);
            if (sampling) mine = stream_part_async<DT, REF, true>(p, row, part, wring, sink, chunks, per);
            else mine = stream_part_async<DT, REF, false>(p, row, part, wring, sink, chunks, per);
            if (lane == 0) {
                lg->count = chunks;
                lg->tiles = per;
            }
        }
        if (lane == 0) sh.sp[b][part] = mine;
    };
    // a row's tail, by the calling warp, once all its parts are delivered
    auto tail_one = [&](uint32_t b) {
        const uint64_t row = row0 + b;
        finalize_row(p, row, kGroupParts, [&](uint32_t q) { return sh.sp[b][q]; }, &sh.res[warp]);
        __syncwarp();
        const RowResult res = sh.res[warp];
        int32_t tok = -1;
        if (!res.status && sampling) {
            const auto* pl = &sh.log[b][res.part];
            if constexpr (ALLOW) tok = pl->count != kLogOverflow ? pick_from_part_log<DT>(p, row, res, pl, wstage) : pick_from_part_scan<DT>(p, row, res);
            else tok = pick_from_chunk_log<DT>(p, row, res, pl);
        }
        if (lane == 0) write_row<DT, REF, ALLOW, false>(p, row, res, tok);
        __syncwarp();
    };

    for (;;) {
        uint32_t t = 0;
        if (lane == 0) t = atomicAdd(&sh.next_ticket, 1u);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= nrows * kGroupParts) break;
        stream_one(t / kGroupParts, t % kGroupParts);
    }
    // every part of every row of the group is delivered: the rows' tails, one warp per row, side by side
    __syncthreads();
    for (uint32_t b = (uint32_t)warp; b < nrows; b += kWarps) tail_one(b);
}

}  // namespace nrl
