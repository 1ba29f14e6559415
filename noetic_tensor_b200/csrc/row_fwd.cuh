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
    uint32_t flags;
    float tau;
};

// elements [begin, end) of part q (block split q / 16, warp q % 16)
__device__ __forceinline__ void part_range(const FwdParams& p, uint32_t q, uint32_t& begin, uint32_t& end) {
    uint32_t split = q / kWarps, w = q % kWarps;
    uint32_t tpw = (p.tiles_per_block + kWarps - 1) / kWarps;
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
            if (ALLOW) k.load(p.allow, row * p.allow_stride + v);
            if (GENERAL && p.add) am.load(p.add, row * p.add_stride + v);
        } else {
            int n = (int)(end - v < (uint32_t)kVec ? end - v : (uint32_t)kVec);
            x.load_scalar(p.logits, e, n);
            if (REF) r.load_scalar(p.ref, e, n);
            if (ALLOW) k.load_scalar(p.allow, row * p.allow_stride + v, n);
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
                bool ok = k.allowed(i);
                z[i] = ok ? z[i] : NRL_NEG_INF;
                if (REF) zr[i] = ok ? zr[i] : NRL_NEG_INF;
            }
        }
    }
};

// fold one vector into a thread's partial
template <bool REF>
__device__ __forceinline__ void accumulate(Partial& a, const float z[8], const float zr[8]) {
    float vmax = z[0];
#pragma unroll
    for (int i = 1; i < 8; i++) vmax = fmax_nan(vmax, z[i]);
    if (vmax != NRL_NEG_INF) {  // something allowed here (or a NaN)
        if (!(vmax <= a.m)) partial_rebase(a.m, a.S, a.W, a.D, fmax_nan(a.m, vmax));
        float s8 = 0.f, w8 = 0.f, d8 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float zc = fmaxf(z[i], -FLT_MAX);  // −inf → finite, so 0·(−inf) never appears
            float t = zc - a.m;
            float e = ex2_approx(t * kLog2e);
            s8 += e;
            w8 = fmaf(e, t, w8);
            if (REF) {
                float d = zc - zr[i];
                if (e > 0.f) d8 = fmaf(e, d, d8);  // a zero-probability token contributes 0
            }
        }
        a.S += s8;
        a.W += w8;
        if (REF) a.D += d8;
    }
    if (REF) {
        float rmax = zr[0];
#pragma unroll
        for (int i = 1; i < 8; i++) rmax = fmax_nan(rmax, zr[i]);
        if (rmax != NRL_NEG_INF) {
            if (!(rmax <= a.mr)) partial_rebase_ref(a.mr, a.Sr, fmax_nan(a.mr, rmax));
            // (zr − mr) first, then the scale: folding mr·log2e into one fma would shift every
            // term of the row by the rounding of that product, and ln Zr with it
            float s8 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) s8 += ex2_approx((zr[i] - a.mr) * kLog2e);
            a.Sr += s8;
        }
    }
}

// A thread block streams its range of one row and leaves 16 part partials in `sp`.
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC>
__device__ __forceinline__ void stream_block(const FwdParams& p, uint64_t row, uint32_t split, Partial* sp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t begin, end;
    part_range(p, split * kWarps + warp, begin, end);
    Partial acc = partial_empty();
    VecLoader<DT, REF, ALLOW, GENERAL, VEC> cur, nxt;
    uint32_t v = begin + lane * kVec;
    bool have = v < end;
    if (have) cur.load(p, row, v, end);
    while (have) {
        uint32_t vn = v + kTile;
        bool have_n = vn < end;
        if (have_n) nxt.load(p, row, vn, end);  // next tile in flight while this one is reduced
        float z[8], zr[8];
        cur.values(p, z, zr);
        accumulate<REF>(acc, z, zr);
        cur = nxt;
        v = vn;
        have = have_n;
    }
    acc = partial_warp_reduce(acc);
    if (lane == 0) sp[warp] = acc;
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
                double dm = (double)a.m - (double)m;
                double c = exp(dm);
                S += c * (double)a.S;
                W += c * ((double)a.W + (double)a.S * dm);
                D += c * (double)a.D;
            }
            if (a.mr != NRL_NEG_INF) Sr += exp((double)a.mr - (double)mr) * (double)a.Sr;
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
                double dm = (double)a.m - (double)m;
                double mass = exp(dm) * (double)a.S;
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
    if (lane == 0) {
        RowResult r;
        r.Z = Z; r.Zr = Srt; r.W = Wt; r.D = Dt;
        r.m = m; r.mr = mr;
        double lnZ = log(Z), lnZr = log(Srt);
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
