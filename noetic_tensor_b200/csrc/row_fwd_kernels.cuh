// The row-forward kernels: the fused one-block-per-row kernel, and the two-stage pair used when
// few long rows are split over several blocks (stage 1 leaves part partials in scratch memory,
// stage 2 merges them and picks the token).
#pragma once
#include "row_fwd.cuh"

namespace nrl {

struct PickShared {
    double warp_tot[kWarps];
    int first_claim[kWarps];
    int last_mass[kWarps];
    uint32_t first_idx[kWarps];
    int32_t token;
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

    // this thread's mass, in element order
    double s = 0.0;
    for (uint32_t v = lo; v < hi; v += kVec) {
        ld.load(p, row, v, hi);
        ld.values(p, z, zr);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float t = fmaxf(z[i], -FLT_MAX) - m;
            float e = ex2_approx(t * kLog2e);
            if (v + i < hi) s += (double)e;
        }
    }
    double incl = warp_scan_incl(s, lane);
    if (lane == 31) ps->warp_tot[warp] = incl;
    __syncthreads();
    double before = 0.0;
    for (int w = 0; w < warp; w++) before += ps->warp_tot[w];
    double excl = before + (incl - s);
    bool claim = s > 0.0 && (excl + s > res.resid);
    uint32_t cb = __ballot_sync(0xffffffffu, claim);
    uint32_t mb = __ballot_sync(0xffffffffu, s > 0.0);
    if (lane == 0) {
        ps->first_claim[warp] = cb ? (warp * 32 + __ffs(cb) - 1) : -1;
        ps->last_mass[warp] = mb ? (warp * 32 + 31 - __clz(mb)) : -1;
    }
    __syncthreads();
    int owner = -1;
    for (int w = 0; w < kWarps && owner < 0; w++) owner = ps->first_claim[w];
    bool take_last = false;
    if (owner < 0) {  // rounding only: no running sum crosses; the last thread with mass ends the row
        take_last = true;
        for (int w = kWarps - 1; w >= 0 && owner < 0; w--) owner = ps->last_mass[w];
    }
    if (tid == owner) {
        double c = excl;
        int32_t tok = -1, last = -1;
        for (uint32_t v = lo; v < hi && tok < 0; v += kVec) {
            ld.load(p, row, v, hi);
            ld.values(p, z, zr);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (tok < 0 && v + i < hi) {
                    float t = fmaxf(z[i], -FLT_MAX) - m;
                    float e = ex2_approx(t * kLog2e);
                    if (e > 0.f) last = (int32_t)(v + i);
                    c += (double)e;
                    if (!take_last && c > res.resid) tok = (int32_t)(v + i);
                }
            }
        }
        ps->token = tok >= 0 ? tok : last;
    }
    __syncthreads();
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
            lp = (z - res.m) - res.lnZ;
            if (REF) rlp = (zr - res.mr) - res.lnZr;
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

// ---- fused: one block per row ---------------------------------------------------------------
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__global__ void __launch_bounds__(kThreads, 2) row_fwd_fused(FwdParams p) {
    __shared__ Partial sp[kWarps];
    __shared__ RowResult res;
    __shared__ PickShared ps;
    const uint64_t row = blockIdx.x;
    stream_block<DT, REF, ALLOW, GENERAL, VEC>(p, row, 0, sp);
    __syncthreads();
    if (threadIdx.x < 32) finalize_row(p, row, kWarps, [&](uint32_t q) { return sp[q]; }, &res);
    __syncthreads();
    const bool pick = !res.status && (p.flags & (NRL_FWD_SAMPLE | NRL_FWD_GREEDY));
    if (pick) pick_token<DT, REF, ALLOW, GENERAL, VEC>(p, row, res, &ps);
    if (threadIdx.x == 0) write_row<DT, REF, ALLOW, GENERAL>(p, row, res, pick ? ps.token : -1);
}

// ---- split, stage 1: a block streams one range of a row and stores its 16 partials ----------
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__global__ void __launch_bounds__(kThreads, 2) row_fwd_parts(FwdParams p) {
    __shared__ Partial sp[kWarps];
    const uint64_t row = blockIdx.x / p.nsplit;
    const uint32_t split = blockIdx.x % p.nsplit;
    stream_block<DT, REF, ALLOW, GENERAL, VEC>(p, row, split, sp);
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
__global__ void __launch_bounds__(kThreads, 2) row_fwd_finish(FwdParams p) {
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
