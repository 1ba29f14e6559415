// The grouped row forward for byte-masked rows (many rows, sampling or given tokens).
//
// In the one-block-per-row kernel a row ends with a tail — merge the part partials, find the
// token, read its logits, write the outputs — during which one warp works through a chain of
// dependent loads while the block's other warps wait, and before it every warp waits for the
// row's slowest part. Here a block takes a group of kGroupRows consecutive rows. Its warps take
// (row, part) tickets from a counter in shared memory, rows in order; a warp streams one part,
// and the warp that delivers a row's last part runs that row's tail while the other warps are
// already streaming the next rows' parts. Each row of the group has its own result buffer, so no
// warp ever waits for another: there is no spin, no barrier after the first, and nothing that
// could hang.
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
constexpr int kGroupRows = NRL_GROUP_ROWS;  // rows per block
constexpr int kPLog = 64;                   // logged batches per part (2048 live vectors)

// What the streaming pass leaves per part for the token pick. A batch is 32 consecutive live
// vectors (vectors with an allowed token) of the part in index order; per batch: the warp's mass
// at maximum cmax, and the batch's first vector as its index within the part. The batch's other
// vectors are found again from the mask.
struct PartLog {
    float mass[kPLog];
    float cmax[kPLog];
    uint16_t first[kPLog];
    uint32_t count;  // batches folded, or kLogOverflow
};

// Lane l holds vector `vv` (or kNoEntry) of one batch; `run` is the mass before the batch.
// Returns the token at which the running mass first exceeds `target`, or −1 if the batch ends
// first (then `run` has the batch added and `last` is the lane's last token with mass, if any).
template <int DT>
__device__ __forceinline__ int32_t scan_batch(const FwdParams& p, uint64_t row, uint32_t vv, uint32_t end, float m, double& run, double target, int32_t& last) {
    typedef VecLoader<DT, false, true, false, true> Loader;
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
            q[j] = (v >= v0 && v < end) ? ldg_stream8(mrow + v) : make_uint2(0u, 0u);
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

// One warp: the token inside part `res.part` from the part's log. Lane c rescales the masses of
// batches c and c + 32 to the row maximum; a scan finds the batch that holds res.resid; that
// batch's vectors are found again from the mask and read again.
template <int DT>
__device__ __forceinline__ int32_t pick_from_part_log(const FwdParams& p, uint64_t row, const RowResult& res, const PartLog* log, uint32_t* slots) {
    const int lane = threadIdx.x & 31;
    uint32_t begin, end;
    part_range(p, res.part, begin, end);
    const uint32_t n = log->count;
    double x[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t c = (uint32_t)lane + 32u * h;
        x[h] = 0.0;
        if (c < n) {
            const float cm = log->cmax[c];
            x[h] = cm == NRL_NEG_INF ? 0.0 : (double)log->mass[c] * (double)expf(cm - res.m);
        }
    }
    const double lo_incl = warp_scan_incl(x[0], lane);
    const double lo_total = __shfl_sync(0xffffffffu, lo_incl, 31);
    const double hi_incl = lo_total + warp_scan_incl(x[1], lane);
    const uint32_t cross_lo = __ballot_sync(0xffffffffu, x[0] > 0.0 && lo_incl > res.resid);
    const uint32_t cross_hi = __ballot_sync(0xffffffffu, x[1] > 0.0 && hi_incl > res.resid);
    const uint32_t has_lo = __ballot_sync(0xffffffffu, x[0] > 0.0);
    const uint32_t has_hi = __ballot_sync(0xffffffffu, x[1] > 0.0);
    if (!(has_lo | has_hi)) return -1;  // the part holds no mass at all
    const bool take_last = !(cross_lo | cross_hi);  // rounding only: the last token with mass of the last batch with mass
    int c;
    if (take_last) c = has_hi ? 32 + (31 - __clz(has_hi)) : 31 - __clz(has_lo);
    else c = cross_lo ? __ffs(cross_lo) - 1 : 32 + __ffs(cross_hi) - 1;
    const double before = c < 32 ? __shfl_sync(0xffffffffu, lo_incl - x[0], c) : __shfl_sync(0xffffffffu, hi_incl - x[1], c - 32);
    const uint32_t v0 = begin + (uint32_t)log->first[c] * kVec;
    const uint32_t vv = regather_batch(p, row, begin, end, v0, slots);
    double run = 0.0;
    int32_t last = -1;
    int32_t tok = scan_batch<DT>(p, row, vv, end, res.m, run, take_last ? 1e300 : res.resid - before, last);
    if (tok < 0) tok = warp_max_i32(last);
    return tok;
}

// One warp, no log (a part that outgrew it): scan the part's vectors 32 at a time, mask bytes
// first, in index order.
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
        int32_t tok = scan_batch<DT>(p, row, mk.any() ? v : kNoEntry, end, res.m, run, res.resid, last);
        if (tok >= 0) return tok;
    }
    return warp_max_i32(last);
}

struct GroupShared {
    Partial sp[kGroupRows][kWarps];
    PartLog log[kGroupRows][kWarps];
    RowResult res[kWarps];
    uint32_t arrived[kGroupRows];  // parts delivered per row
    uint32_t next_ticket;
};

// With a reference stream the loop holds two more 16-byte loads per vector in flight: three blocks
// per SM (80 registers per thread) measured faster than four (64, with spills).
#ifndef NRL_GROUP_BLOCKS_REF
#define NRL_GROUP_BLOCKS_REF 3
#endif
template <int DT, bool REF>
__global__ void __launch_bounds__(kThreads, REF ? NRL_GROUP_BLOCKS_REF : 1024 / kThreads) row_fwd_grouped(FwdParams p) {
    __shared__ GroupShared sh;
    __shared__ __align__(16) uint32_t queue[kWarps * kQueue];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int b = 0; b < kGroupRows; b++) sh.arrived[b] = 0u;
        sh.next_ticket = 0u;
    }
    __syncthreads();
    const uint64_t row0 = (uint64_t)blockIdx.x * kGroupRows;
    const uint64_t left = p.rows - row0;
    const uint32_t tickets = (uint32_t)(left < (uint64_t)kGroupRows ? left : (uint64_t)kGroupRows) * kWarps;
    const bool sampling = (p.flags & NRL_FWD_SAMPLE) != 0;
    uint32_t* wq = queue + warp * kQueue;

    for (;;) {
        uint32_t t = 0;
        if (lane == 0) t = atomicAdd(&sh.next_ticket, 1u);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= tickets) break;
        const uint32_t b = t / kWarps, part = t % kWarps;
        const uint64_t row = row0 + b;

        PartLog* lg = &sh.log[b][part];
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
        Partial mine;
        if (sampling) mine = stream_part_compact<DT, REF, true>(p, row, part, wq, sink, batches);
        else mine = stream_part_compact<DT, REF, false>(p, row, part, wq, sink, batches);
        if (lane == 0) {
            sh.sp[b][part] = mine;
            lg->count = batches <= (uint32_t)kPLog ? batches : kLogOverflow;
        }
        __syncwarp();
        __threadfence_block();  // the part's results are visible before its arrival is
        uint32_t before = 0;
        if (lane == 0) before = atomicAdd(&sh.arrived[b], 1u);
        before = __shfl_sync(0xffffffffu, before, 0);
        if (before != kWarps - 1) continue;

        // this warp delivered the row's last part: the row's tail
        __threadfence_block();
        finalize_row(p, row, kWarps, [&](uint32_t q) { return sh.sp[b][q]; }, &sh.res[warp]);
        __syncwarp();
        const RowResult res = sh.res[warp];
        int32_t tok = -1;
        if (!res.status && sampling) {
            const PartLog* pl = &sh.log[b][res.part];
            tok = pl->count != kLogOverflow ? pick_from_part_log<DT>(p, row, res, pl, wq) : pick_from_part_scan<DT>(p, row, res);
        }
        if (lane == 0) write_row<DT, REF, true, false>(p, row, res, tok);
        __syncwarp();
    }
}

}  // namespace nrl
