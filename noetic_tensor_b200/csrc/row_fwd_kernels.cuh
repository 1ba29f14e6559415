// The row-forward kernels: the fused one-block-per-row kernel, and the two-stage pair used when
// few long rows are split over several blocks (stage 1 leaves part partials in scratch memory,
// stage 2 merges them and picks the token).
#pragma once
#include <type_traits>

#include "row_fwd.cuh"

namespace nrl {

struct PickShared {
    double warp_tot[kWarps];
    int first_claim[kWarps];
    int last_mass[kWarps];
    uint32_t first_idx[kWarps];
    int32_t token;
    int32_t last_token;
    uint32_t chunk_a, chunk_b;  // unmasked path: the chunk warp 0 found, re-read by the whole block
    double chunk_resid;
    float z_tok, zr_tok;
};

template <int DT, bool REF, bool ALLOW, bool GENERAL>
__device__ __forceinline__ void load_one(const FwdParams& p, uint64_t row, uint32_t v, float& z, float& zr) {
    VecLoader<DT, REF, ALLOW, GENERAL, false> one;
    one.load(p, row, v, v + 1);
    float zz[8], rr[8];
    one.values(p, zz, rr);
    z = zz[0];
    zr = REF ? rr[0] : 0.f;
}

// Sampling inside part `res.part`: the first element, in index order, at which the running mass
// exceeds res.resid. The part is covered in rounds of kThreads·64 elements; in a round thread j
// owns the 8 vectors [j·64, j·64+64) of the round, so (round, thread, vector, element) is index
// order. A thread keeps the masses of its 8 vectors; a block scan of the thread totals finds the
// owner thread, which finds its vector from the kept masses and re-reads only that one vector.
// With a byte mask, the mask bytes are read first and logits only for vectors that allow a token.
constexpr int kPickVec = 8;

template <int DT, bool ALLOW, bool GENERAL, bool VEC>
__device__ __forceinline__ float vector_mass(const FwdParams& p, const VecLoader<DT, false, ALLOW, GENERAL, VEC>& ld, float m, uint32_t v, uint32_t hi) {
    float z[8], zr[8];
    ld.values(p, z, zr);
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float t = fmaxf(z[i], -FLT_MAX) - m;
        float e = ex2_approx(t * kLog2e);
        if (v + i < hi) s += (double)e;
    }
    return (float)s;
}

template <int DT, bool ALLOW, bool GENERAL, bool VEC>
__device__ __forceinline__ void pick_sample(const FwdParams& p, uint64_t row, uint32_t a, uint32_t b, float m, double resid, PickShared* ps) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    typedef VecLoader<DT, false, ALLOW, GENERAL, VEC> Loader;
    const uint8_t* mrow = ALLOW ? p.allow + row * p.allow_stride : nullptr;
    double base = 0.0;  // mass of the rounds before this one (block-uniform)
    if (tid == 0) ps->last_token = -1;
    for (uint32_t r0 = a; r0 < b; r0 += kThreads * kPickVec * kVec) {
        const uint32_t lo = r0 + (uint32_t)tid * (kPickVec * kVec);
        float vm[kPickVec];
        // mask bytes first: an excluded vector costs 8 bytes, not 8 logits
        bool live[kPickVec];
#pragma unroll
        for (int k = 0; k < kPickVec; k++) {
            uint32_t v = lo + k * kVec;
            live[k] = v < b;
            if (ALLOW && VEC && !GENERAL) {
                RawMask mk;
                mk.q = make_uint2(0u, 0u);
                if (live[k]) mk.load(mrow, v);
                live[k] = mk.any();
            }
        }
#pragma unroll
        for (int g = 0; g < kPickVec; g += 4) {
            Loader ld[4];
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (live[g + k]) ld[k].load(p, row, lo + (g + k) * kVec, b);
#pragma unroll
            for (int k = 0; k < 4; k++) vm[g + k] = live[g + k] ? vector_mass<DT, ALLOW, GENERAL, VEC>(p, ld[k], m, lo + (g + k) * kVec, b) : 0.f;
        }
        double s = 0.0;
#pragma unroll
        for (int k = 0; k < kPickVec; k++) s += (double)vm[k];
        double incl = warp_scan_incl(s, lane);
        __syncthreads();  // the previous round's reads of the shared slots are done
        if (lane == 31) ps->warp_tot[warp] = incl;
        __syncthreads();
        double before = base, total = base;
        for (int w = 0; w < kWarps; w++) {
            if (w < warp) before += ps->warp_tot[w];
            total += ps->warp_tot[w];
        }
        double excl = before + (incl - s);
        bool claim = s > 0.0 && (excl + s > resid);
        uint32_t cb = __ballot_sync(0xffffffffu, claim);
        uint32_t mb = __ballot_sync(0xffffffffu, s > 0.0);
        if (lane == 0) {
            ps->first_claim[warp] = cb ? (warp * 32 + __ffs(cb) - 1) : -1;
            ps->last_mass[warp] = mb ? (warp * 32 + 31 - __clz(mb)) : -1;
        }
        __syncthreads();
        int owner = -1, last_owner = -1;
        for (int w = 0; w < kWarps; w++) {
            if (owner < 0) owner = ps->first_claim[w];
            if (ps->last_mass[w] >= 0) last_owner = ps->last_mass[w];
        }
        // the thread that ends the row if rounding leaves no crossing: the last one with mass
        const bool crossing = owner >= 0;
        if (!crossing) owner = last_owner;
        if (tid == owner) {
            // find the vector from the kept masses, then walk its 8 elements
            double c = excl;
            int kk = -1, klast = -1;
#pragma unroll
            for (int k = 0; k < kPickVec; k++) {
                if (vm[k] > 0.f) {
                    klast = k;
                    if (kk < 0 && crossing && c + (double)vm[k] > resid) kk = k;
                    if (kk < 0) c += (double)vm[k];
                }
            }
            const bool take_last = kk < 0;
            if (take_last) kk = klast;
            if (kk >= 0) {
                if (take_last) c = 0.0;  // irrelevant: the last element with mass is taken
                uint32_t v = lo + kk * kVec;
                Loader one;
                one.load(p, row, v, b);
                float z[8], zr[8];
                one.values(p, z, zr);
                int32_t tok = -1, last = -1;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (v + i < b) {
                        float t = fmaxf(z[i], -FLT_MAX) - m;
                        float e = ex2_approx(t * kLog2e);
                        if (e > 0.f) last = (int32_t)(v + i);
                        c += (double)e;
                        if (tok < 0 && !take_last && c > resid) tok = (int32_t)(v + i);
                    }
                }
                if (crossing) ps->token = tok >= 0 ? tok : last;
                else ps->last_token = last;
            }
        }
        __syncthreads();
        if (crossing) return;       // block-uniform: ps->token is set
        base = total;
    }
    // no crossing in any round (rounding only): the last token with mass seen
    if (tid == 0) ps->token = ps->last_token;
    __syncthreads();
}

// Sampling from the log the streaming pass left (fused kernel): warp 0 alone finds the chunk of
// part `res.part` that holds res.resid from the logged chunk masses, reads that one chunk again
// (up to tiles_per_chunk vectors per lane on the unmasked path, one queued vector per lane on
// the masked path) and walks to the token. Index order inside a chunk is (tile, lane, element).
// Returns false (block-uniform, nothing written) if the part outgrew the log.
template <int DT, bool ALLOW, class Log>
__device__ __forceinline__ bool pick_logged(const FwdParams& p, uint64_t row, const RowResult& res, const Log* log, PickShared* ps) {
    typedef VecLoader<DT, false, ALLOW, false, true> Loader;
    const uint32_t w = res.part;
    const uint32_t n = log->count[w];
    if (n == kLogOverflow) return false;
    if (threadIdx.x >= 32) return true;
    const int lane = threadIdx.x;
    const float m = res.m;
    uint32_t begin, end;
    part_range(p, w, begin, end);
    // the chunk: running prefix of chunk masses at the row maximum, lower chunks first
    double prefix = 0.0, r2 = 0.0;
    int cstar = -1, clast = -1;
    for (uint32_t c = 0; c < n; c++) {
        const float cm = log->cmax[w][c];
        double x = cm == NRL_NEG_INF ? 0.0 : (double)log->mass[w][c][lane] * (double)expf(cm - m);
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
        if (x > 0.0) clast = (int)c;
        if (cstar < 0 && prefix + x > res.resid) {
            cstar = (int)c;
            r2 = res.resid - prefix;
        }
        if (cstar < 0) prefix += x;
    }
    const bool take_last = cstar < 0;  // rounding only: the last token with mass of the last chunk with mass
    if (take_last) cstar = clast;
    if (cstar < 0) {  // the part holds no mass at all: no token
        if (lane == 0) {
            ps->token = -1;
            ps->chunk_a = ps->chunk_b = 0;
            ps->chunk_resid = 0.0;
        }
        return true;
    }
    if constexpr (!ALLOW) {
        // unmasked path: hand the chunk's element range to the whole block (one vector per thread
        // when a chunk is 8 tiles), which scans it like a small part
        if (lane == 0) {
            const uint32_t tiles = log->tiles_per_chunk[w];
            const uint32_t ca = begin + (uint32_t)cstar * tiles * kTile;
            const uint32_t cb = ca + tiles * kTile;
            ps->chunk_a = ca < end ? ca : end;
            ps->chunk_b = cb < end ? cb : end;
            ps->chunk_resid = take_last ? 1e300 : r2;
        }
        return true;
    } else {
    // masked path: the chunk is one batch, lane l holds its queued vector
    double run = 0.0;
    int32_t token = -1, last = -1;
    {
        Loader ld;
        const uint32_t vv = log->entry[w][cstar][lane];
        if (vv != kNoEntry) ld.load(p, row, vv, end);
        float e[8];
        double s = 0.0;
        if (vv != kNoEntry) {
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
        const bool mine = !take_last && s > 0.0 && run + incl > r2;
        const uint32_t ball = __ballot_sync(0xffffffffu, mine);
        if (ball) {
            const int owner = __ffs(ball) - 1;
            int32_t tok = -1;
            if (lane == owner) {
                double c = run + (incl - s);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    c += (double)e[i];
                    if (tok < 0 && e[i] > 0.f && c > r2) tok = (int32_t)(vv + i);
                }
                if (tok < 0) tok = last;  // rounding inside the vector
            }
            token = __shfl_sync(0xffffffffu, tok, owner);
        }
    }
    if (token < 0) {  // no crossing (rounding): the last token with mass in the batch
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            int32_t o = __shfl_xor_sync(0xffffffffu, last, s);
            last = o > last ? o : last;
        }
        token = last;
    }
    if (lane == 0) ps->token = token;
    return true;
    }
}

// All threads of the block: find the token inside part `res.part`.
//   sampling: the first element, in index order, at which the running mass exceeds res.resid;
//   greedy:   the first element equal to the row maximum.
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__device__ __forceinline__ void pick_token(const FwdParams& p, uint64_t row, const RowResult& res, PickShared* ps) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool greedy = (p.flags & NRL_FWD_GREEDY) != 0;
    uint32_t a, b;
    part_range(p, res.part, a, b);
    uint32_t len = b - a;
    uint32_t per = (len + kThreads - 1) / kThreads;
    per = (per + kVec - 1) / kVec * kVec;
    uint32_t lo = a + (uint32_t)tid * per;
    uint32_t hi = lo + per;
    if (lo > b) lo = b;
    if (hi > b) hi = b;
    const float m = res.m;
    VecLoader<DT, false, ALLOW, GENERAL, VEC> ld;
    float z[8], zr[8];

    if (greedy) {
        uint32_t first = 0xffffffffu;
        for (uint32_t v = lo; v < hi; v += kVec) {
            ld.load(p, row, v, hi);
            ld.values(p, z, zr);
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (first == 0xffffffffu && v + i < hi && z[i] == m) first = v + i;
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            uint32_t o = __shfl_xor_sync(0xffffffffu, first, s);
            first = o < first ? o : first;
        }
        if (lane == 0) ps->first_idx[warp] = first;
        __syncthreads();
        if (tid == 0) {
            uint32_t f = 0xffffffffu;
            for (int w = 0; w < kWarps; w++) f = ps->first_idx[w] < f ? ps->first_idx[w] : f;
            ps->token = (int32_t)f;
        }
        __syncthreads();
        return;
    }

    pick_sample<DT, ALLOW, GENERAL, VEC>(p, row, a, b, res.m, res.resid, ps);
}

// Thread 0 writes the row's outputs.
template <int DT, bool REF, bool ALLOW, bool GENERAL>
__device__ __forceinline__ void write_row(const FwdParams& p, uint64_t row, const RowResult& res, int32_t tok) {
    const float qnan = __int_as_float(0x7fc00000);
    uint32_t status = res.status;
    bool want_tok = (p.flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY | NRL_FWD_TOKENS_IN)) != 0;
    float lp = qnan, rlp = qnan;
    if (!status && want_tok) {
        if (p.flags & NRL_FWD_TOKENS_IN) tok = p.tokens[row];
        if (tok < 0 || (uint32_t)tok >= p.V) {
            status |= 4u;  // a token outside the vocabulary
        } else {
            float z, zr;
            load_one<DT, REF, ALLOW, GENERAL>(p, row, (uint32_t)tok, z, zr);
            // an excluded token (−inf logit, or masked out: −FLT_MAX inside the kernels) has log-prob −inf
            lp = z <= -FLT_MAX ? NRL_NEG_INF : (z - res.m) - res.lnZ;
            if (REF) rlp = zr <= -FLT_MAX ? NRL_NEG_INF : (zr - res.mr) - res.lnZr;
        }
    }
    bool bad = (status & 3u) != 0;
    if (p.tokens && (p.flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY))) p.tokens[row] = bad ? -1 : tok;
    if (p.logp) p.logp[row] = lp;
    if (p.ref_logp) p.ref_logp[row] = rlp;
    if (p.kl) p.kl[row] = bad ? qnan : res.kl;
    if (p.entropy) p.entropy[row] = bad ? qnan : res.ent;
    if (p.rowstats) {
        float4 st = bad ? make_float4(qnan, qnan, qnan, qnan) : make_float4(res.m, res.lnZ, res.mr, res.lnZr);
        reinterpret_cast<float4*>(p.rowstats)[row] = st;
    }
    if (p.status) p.status[row] = (uint8_t)status;
}

// Streams a block's range of a row: byte-masked rows on the vectorised fast path go through the
// compacting scan, unmasked ones through the asynchronous ring, everything else through the plain
// tile loop. With LOG the fast paths also leave the sampling log for pick_logged.
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
struct FastPath {
    static constexpr bool compact = ALLOW && VEC && !GENERAL;
    static constexpr bool ring = !ALLOW && VEC && !GENERAL;
    typedef typename std::conditional<compact, CompactLog, DenseLog>::type Log;
};

// the staging area a fast path needs in shared memory: the vector queue or the copy ring
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
struct Stage {
    typedef FastPath<DT, REF, ALLOW, GENERAL, VEC> F;
    static constexpr int words = F::compact ? kWarps * kQueue : (F::ring ? kWarps * kRingRows * 32 * 4 : 4);
};

template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC, bool LOG>
__device__ __forceinline__ void stream_row(const FwdParams& p, uint64_t row, uint32_t split, Partial* sp, uint32_t* stage, typename FastPath<DT, REF, ALLOW, GENERAL, VEC>::Log* log) {
    typedef FastPath<DT, REF, ALLOW, GENERAL, VEC> F;
    if constexpr (F::compact) {
        stream_block_compact<DT, REF, LOG>(p, row, split, sp, stage, log);
    } else if constexpr (F::ring) {
        stream_block_async<DT, REF, LOG>(p, row, split, sp, reinterpret_cast<uint4*>(stage), log);
    } else {
        stream_block<DT, REF, ALLOW, GENERAL, VEC>(p, row, split, sp);
    }
}

// ---- fused: one block per row ---------------------------------------------------------------
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) row_fwd_fused(FwdParams p) {
    typedef FastPath<DT, REF, ALLOW, GENERAL, VEC> F;
    // The log pays off on the masked path (one queued vector per lane to re-read). On the unmasked
    // path the whole-part scan by the full block measured faster, so that path does not log.
    constexpr bool kLogged = F::compact;
    __shared__ Partial sp[kWarps];
    __shared__ RowResult res;
    __shared__ PickShared ps;
    __shared__ typename std::conditional<kLogged, typename F::Log, int>::type slog;
    __shared__ __align__(16) uint32_t stage[Stage<DT, REF, ALLOW, GENERAL, VEC>::words];
    const uint64_t row = blockIdx.x;
    const bool sampling = (p.flags & NRL_FWD_SAMPLE) != 0;
    if constexpr (kLogged) {
        if (sampling) stream_row<DT, REF, ALLOW, GENERAL, VEC, true>(p, row, 0, sp, stage, &slog);
        else stream_row<DT, REF, ALLOW, GENERAL, VEC, false>(p, row, 0, sp, stage, &slog);
    } else {
        stream_row<DT, REF, ALLOW, GENERAL, VEC, false>(p, row, 0, sp, stage, nullptr);
    }
    __syncthreads();
    if (threadIdx.x < 32) finalize_row(p, row, kWarps, [&](uint32_t q) { return sp[q]; }, &res);
    __syncthreads();
    const bool pick = !res.status && (p.flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY));
    if (pick) {
        bool done = false;
        if constexpr (kLogged) {
            if (sampling) {
                done = pick_logged<DT, ALLOW>(p, row, res, &slog, &ps);
                if constexpr (F::ring) {
                    if (done) {
                        __syncthreads();
                        pick_sample<DT, ALLOW, GENERAL, VEC>(p, row, ps.chunk_a, ps.chunk_b, res.m, ps.chunk_resid, &ps);
                    }
                }
            }
        }
        if (!done) pick_token<DT, REF, ALLOW, GENERAL, VEC>(p, row, res, &ps);
        __syncthreads();
    }
    if (threadIdx.x == 0) write_row<DT, REF, ALLOW, GENERAL>(p, row, res, pick ? ps.token : -1);
}

// ---- split, stage 1: a block streams one range of a row and stores its 16 partials ----------
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) row_fwd_parts(FwdParams p) {
    __shared__ Partial sp[kWarps];
    const uint64_t row = blockIdx.x / p.nsplit;
    const uint32_t split = blockIdx.x % p.nsplit;
    __shared__ __align__(16) uint32_t stage[Stage<DT, REF, ALLOW, GENERAL, VEC>::words];
    stream_row<DT, REF, ALLOW, GENERAL, VEC, false>(p, row, split, sp, stage, nullptr);
    __syncthreads();
    if (threadIdx.x < kWarps) {
        Partial a = sp[threadIdx.x];
        float* o = p.parts + ((row * p.nsplit + split) * kWarps + threadIdx.x) * kPartFloats;
        reinterpret_cast<float4*>(o)[0] = make_float4(a.m, a.S, a.W, a.D);
        reinterpret_cast<float4*>(o)[1] = make_float4(a.mr, a.Sr, 0.f, 0.f);
    }
}

// ---- split, stage 2: merge a row's partials, pick the token, write the outputs --------------
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) row_fwd_finish(FwdParams p) {
    __shared__ RowResult res;
    __shared__ PickShared ps;
    const uint64_t row = blockIdx.x;
    const uint32_t nparts = p.nsplit * kWarps;
    const float* base = p.parts + row * nparts * kPartFloats;
    if (threadIdx.x < 32) {
        finalize_row(p, row, nparts, [&](uint32_t q) {
            float4 a = reinterpret_cast<const float4*>(base + (uint64_t)q * kPartFloats)[0];
            float4 b = reinterpret_cast<const float4*>(base + (uint64_t)q * kPartFloats)[1];
            Partial r;
            r.m = a.x; r.S = a.y; r.W = a.z; r.D = a.w; r.mr = b.x; r.Sr = b.y;
            return r;
        }, &res);
    }
    __syncthreads();
    const bool pick = !res.status && (p.flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY));
    if (pick) pick_token<DT, REF, ALLOW, GENERAL, VEC>(p, row, res, &ps);
    if (threadIdx.x == 0) write_row<DT, REF, ALLOW, GENERAL>(p, row, res, pick ? ps.token : -1);
}

}  // namespace nrl
