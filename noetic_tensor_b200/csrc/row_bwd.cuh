// Row backward: d(logits) [rows, V] f32 in one streaming pass from the logits and the per-row
// statistics the forward saved. Purely element-wise given those statistics, so there is no
// reduction here and nothing to order; the pass is bound by the 4-byte-per-element write.
#pragma once
#include "row_fwd.cuh"

namespace nrl {

struct BwdParams {
    FwdParams in;  // logits / ref / masks / V / rows / tau (the forward's view of the inputs)
    const int32_t* tokens;
    const float* rowstats;
    const float* kl;
    const float* entropy;
    const float* g_logp;
    const float* g_kl;
    const float* g_ent;
    const float* g_uni;  // upstream of −mean_v log π_v (label smoothing), or null
    float* d_logits;     // may be null when d_ref is given
    float* d_ref;        // gradient w.r.t. the reference logits of the KL term, or null
    uint32_t chunks_per_row;  // blocks per row
    uint32_t accumulate;      // add into the outputs
};

// 8 consecutive f32 of a gradient row: two 16-byte streaming stores, or element stores on a ragged tail
__device__ __forceinline__ void store_grad8(float* out, uint32_t v, uint32_t v_end, const float g[8], bool vec_out) {
    if (vec_out) {
        stg_stream16(out + v, g[0], g[1], g[2], g[3]);
        stg_stream16(out + v + 4, g[4], g[5], g[6], g[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (v + i < v_end) out[v + i] = g[i];
    }
}

constexpr int kBwdThreads = 256;

// EXTRA: the call uses `accumulate`, the label-smoothing upstream or the reference-side gradient;
// without it the kernel is compiled with none of their code.
template <int DT, bool REF, bool ALLOW, bool GENERAL, bool VEC, bool EXTRA>
__global__ void __launch_bounds__(kBwdThreads, 4) row_bwd_kernel(BwdParams p) {
    const FwdParams& f = p.in;
    const uint64_t row = blockIdx.x / p.chunks_per_row;
    const uint32_t chunk = blockIdx.x % p.chunks_per_row;
    const uint32_t V = f.V;
    // this block's range of the row, in whole vectors
    const uint32_t nvec = (V + kVec - 1) / kVec;
    const uint32_t vec_per = (nvec + p.chunks_per_row - 1) / p.chunks_per_row;
    const uint32_t v_begin = min(chunk * vec_per, nvec) * kVec;
    const uint32_t v_end = min(min((chunk + 1) * vec_per, nvec) * kVec, V);
    float* out = (!EXTRA || p.d_logits) ? p.d_logits + row * V : nullptr;
    float* out_ref = (EXTRA && REF && p.d_ref) ? p.d_ref + row * V : nullptr;
    const bool accumulate = EXTRA && p.accumulate != 0u;

    const float glp = p.g_logp ? p.g_logp[row] : 0.f;
    const float gkl = (REF && p.g_kl) ? p.g_kl[row] : 0.f;
    const float gen = p.g_ent ? p.g_ent[row] : 0.f;
    const float gun = (EXTRA && p.g_uni) ? p.g_uni[row] : 0.f;
    const float gun_v = gun != 0.f ? __fdiv_rn(gun, (float)V) : 0.f;
    const bool vec_out = VEC && (((reinterpret_cast<uintptr_t>(p.d_logits) | reinterpret_cast<uintptr_t>(p.d_ref)) & 15u) == 0);

    if (glp == 0.f && gkl == 0.f && gen == 0.f && gun == 0.f) {
        if (accumulate) return;  // adding exact zeros
        // an unscored position: exact zeros, the inputs are not read
        const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (uint32_t v = v_begin + threadIdx.x * kVec; v < v_end; v += kBwdThreads * kVec) {
            if (out) store_grad8(out, v, v_end, zero, vec_out);
            if (out_ref) store_grad8(out_ref, v, v_end, zero, vec_out);
        }
        return;
    }

    const float4 st = reinterpret_cast<const float4*>(p.rowstats)[row];
    const float m = st.x, lnZ = st.y, mr = st.z, lnZr = st.w;
    const float klv = (REF && p.kl && gkl != 0.f) ? p.kl[row] : 0.f;
    const float hv = (p.entropy && gen != 0.f) ? p.entropy[row] : 0.f;
    const int32_t tok = (p.tokens && glp != 0.f) ? p.tokens[row] : -1;

    VecLoader<DT, REF, ALLOW, GENERAL, VEC> ld;
    for (uint32_t v = v_begin + threadIdx.x * kVec; v < v_end; v += kBwdThreads * kVec) {
        if constexpr (ALLOW && VEC && !GENERAL) {
            // an excluded vector has zero gradient whatever its logits are: only its 8 mask bytes are read
            RawMask mk;
            mk.load(f.allow + row * f.allow_stride, v);
            const bool holds_token = tok >= (int32_t)v && tok < (int32_t)(v + kVec);  // its entry gets g_lp even if excluded
            if (!mk.any() && !holds_token) {
                if (accumulate) continue;
                const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (out) store_grad8(out, v, v_end, zero, vec_out);
                if (out_ref) store_grad8(out_ref, v, v_end, zero, vec_out);
                continue;
            }
        }
        ld.load(f, row, v, v_end);
        float z[8], zr[8], g[8], gr[8];
        ld.values(f, z, zr);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float zc = fmaxf(z[i], -FLT_MAX);
            float lp = (zc - m) - lnZ;
            float pi = ex2_approx(lp * kLog2e);
            float c = -glp;                                   // d logp / dz_j = 1[j = tok] − π_j
            float lr = 0.f;
            if (REF) {
                lr = (zr[i] - mr) - lnZr;
                c = fmaf(gkl, (lp - lr) - klv, c);            // d KL / dz_j = π_j (log π_j − log ρ_j − KL)
            }
            c = fmaf(-gen, lp + hv, c);                       // d H / dz_j = −π_j (log π_j + H)
            if (EXTRA) c += gun;                              // d(−mean_v log π_v) / dz_j = π_j − 1/V
            float d = pi > 0.f ? pi * c : 0.f;                // a zero-probability token gets exactly 0
            if (EXTRA) d -= gun_v;
            if ((int32_t)(v + i) == tok) d += glp;
            if (GENERAL && f.tau != 1.0f) d = __fdiv_rn(d, f.tau);
            g[i] = d;
            if (EXTRA && REF && out_ref) {                    // d KL / dzr_j = ρ_j − π_j (block-uniform branch)
                float dr = gkl * (ex2_approx(lr * kLog2e) - pi);
                if (GENERAL && f.tau != 1.0f) dr = __fdiv_rn(dr, f.tau);
                gr[i] = dr;
            }
        }
        if (out) {
            if (accumulate) {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if (v + i < v_end) g[i] += out[v + i];
            }
            store_grad8(out, v, v_end, g, vec_out);
        }
        if (EXTRA && REF && out_ref) {
            if (accumulate) {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if (v + i < v_end) gr[i] += out_ref[v + i];
            }
            store_grad8(out_ref, v, v_end, gr, vec_out);
        }
    }
}

// ---- the common case: vectorised inputs, no temperature / additive mask, none of the extras --------
//
// The gradient is f32, so a lane that owned 8 consecutive elements would write 32 bytes with
// two 16-byte stores, and each warp-wide store would touch every 32-byte sector of a kilobyte
// but fill only half of it. Here a warp owns a 256-element tile as two 128-element halves and a
// lane takes 4 consecutive elements of each (element 4·lane and 128 + 4·lane of the tile): every
// warp-wide store, and every load of f32 logits, covers 512 contiguous bytes. bf16 logits arrive
// as 8-byte loads (256 contiguous bytes per warp), mask bytes as 4-byte loads.

template <int DT>
struct Piece {  // 4 consecutive elements of one stream
    uint4 q;    // bf16: x, y hold them; f32: all four words
    __device__ __forceinline__ void load(const void* base, uint64_t elem) {
        if constexpr (DT == NRL_BF16) {
            const uint2 h = ldg_stream8((const uint16_t*)base + elem);
            q = make_uint4(h.x, h.y, 0u, 0u);
        } else {
            q = ldg_stream16((const float*)base + elem);
        }
    }
    __device__ __forceinline__ void unpack(float z[4]) const {
        if constexpr (DT == NRL_BF16) {
            z[0] = bf16_lo(q.x); z[1] = bf16_hi(q.x); z[2] = bf16_lo(q.y); z[3] = bf16_hi(q.y);
        } else {
            z[0] = __uint_as_float(q.x); z[1] = __uint_as_float(q.y); z[2] = __uint_as_float(q.z); z[3] = __uint_as_float(q.w);
        }
    }
};

template <int DT, bool REF, bool ALLOW>
__global__ void __launch_bounds__(kBwdThreads, 4) row_bwd_split_kernel(BwdParams p) {
    const FwdParams& f = p.in;
    const uint64_t row = blockIdx.x / p.chunks_per_row;
    const uint32_t chunk = blockIdx.x % p.chunks_per_row;
    const uint32_t V = f.V;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this block's range of the row, in whole tiles
    const uint32_t ntiles = (V + kTile - 1) / kTile;
    const uint32_t tiles_per = (ntiles + p.chunks_per_row - 1) / p.chunks_per_row;
    const uint32_t t_begin = min(chunk * tiles_per, ntiles) * kTile;
    const uint32_t t_end = min(min((chunk + 1) * tiles_per, ntiles) * kTile, V);
    float* out = p.d_logits + row * V;
    constexpr uint32_t kHalf = kTile / 2, kStep = (kBwdThreads / 32) * kTile;

    const float glp = p.g_logp ? p.g_logp[row] : 0.f;
    const float gkl = (REF && p.g_kl) ? p.g_kl[row] : 0.f;
    const float gen = p.g_ent ? p.g_ent[row] : 0.f;
    if (glp == 0.f && gkl == 0.f && gen == 0.f) {
        // an unscored position: exact zeros, the inputs are not read
        for (uint32_t t = t_begin + warp * kTile; t < t_end; t += kStep) {
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const uint32_t e = t + k * kHalf + lane * 4;
                if (e < t_end) stg_stream16(out + e, 0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }
    const float4 st = reinterpret_cast<const float4*>(p.rowstats)[row];
    const float m = st.x, lnZ = st.y, mr = st.z, lnZr = st.w;
    const float klv = (REF && p.kl && gkl != 0.f) ? p.kl[row] : 0.f;
    const float hv = (p.entropy && gen != 0.f) ? p.entropy[row] : 0.f;
    const int32_t tok = (p.tokens && glp != 0.f) ? p.tokens[row] : -1;
    const uint8_t* mrow = ALLOW ? f.allow + row * f.allow_stride : nullptr;

    for (uint32_t t = t_begin + warp * kTile; t < t_end; t += kStep) {
        uint32_t e[2], mk[2];
        bool live[2];
        Piece<DT> x[2], r[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            e[k] = t + k * kHalf + lane * 4;
            mk[k] = 0xffffffffu;
            if (ALLOW) mk[k] = e[k] < t_end ? ldg_mask4(mrow, e[k]) : 0u;
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            // an excluded piece has zero gradient whatever its logits are (only its mask bytes are
            // read), unless it holds the token, whose entry gets g_lp even if excluded
            const bool holds_token = tok >= (int32_t)e[k] && tok < (int32_t)(e[k] + 4);
            live[k] = e[k] < t_end && (mk[k] != 0u || holds_token);
            if (live[k]) {
                x[k].load(f.logits, row * V + e[k]);
                if (REF) r[k].load(f.ref, row * V + e[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            if (e[k] >= t_end) continue;
            float g[4] = {0.f, 0.f, 0.f, 0.f};
            if (live[k]) {
                float z[4], zr[4];
                x[k].unpack(z);
                if (REF) r[k].unpack(zr);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const bool ok = !ALLOW || ((mk[k] >> (8 * i)) & 0xffu) != 0u;
                    const float zc = ok ? fmaxf(z[i], -FLT_MAX) : -FLT_MAX;
                    const float lp = (zc - m) - lnZ;
                    const float pi = ex2_approx(lp * kLog2e);
                    float c = -glp;                                   // d logp / dz_j = 1[j = tok] − π_j
                    if (REF) {
                        const float zrc = ok ? zr[i] : -FLT_MAX;
                        c = fmaf(gkl, (lp - ((zrc - mr) - lnZr)) - klv, c);  // d KL / dz_j = π_j (log π_j − log ρ_j − KL)
                    }
                    c = fmaf(-gen, lp + hv, c);                       // d H / dz_j = −π_j (log π_j + H)
                    float d = pi > 0.f ? pi * c : 0.f;                // a zero-probability token gets exactly 0
                    if ((int32_t)(e[k] + i) == tok) d += glp;
                    g[i] = d;
                }
            }
            stg_stream16(out + e[k], g[0], g[1], g[2], g[3]);
        }
    }
}

// ---- rows under an allow-mask that excludes most of the vocabulary ------------------------------------
//
// Under a grammar mask most 8-element vectors are excluded whole, and the few live ones are
// scattered: in the kernels above a warp runs the whole gradient arithmetic for the two or three
// lanes that hold a live vector (9 of 32 threads active on the benchmark's masks) and waits for
// the mask, then for the logits, one tile at a time. Here a warp works like the forward's
// compacting loop: it scans its range's mask four tiles at a time (the next four in flight),
// stores the zeros of excluded vectors at once — as 16-byte pieces laid out so that every
// warp-wide store fills whole sectors — and queues the live vectors in shared memory; whenever 32
// are queued every lane takes one, its loads fly while the previous batch's gradients are
// computed, and each lane writes its 32 bytes. The values are the kernels' above, bit for bit
// (the same expression per element).
constexpr int kBwdQueue = 256;
constexpr int kBwdAhead = 4;

template <int DT, bool REF>
__global__ void __launch_bounds__(kBwdThreads, 4) row_bwd_compact_kernel(BwdParams p) {
    __shared__ uint32_t queues[kBwdThreads / 32][kBwdQueue];
    const FwdParams& f = p.in;
    const uint64_t row = blockIdx.x / p.chunks_per_row;
    const uint32_t chunk = blockIdx.x % p.chunks_per_row;
    const uint32_t V = f.V;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t lt = (1u << lane) - 1u;
    // this warp's range of the row, in whole tiles
    const uint32_t ntiles = (V + kTile - 1) / kTile;
    const uint32_t nparts = p.chunks_per_row * (kBwdThreads / 32);
    const uint32_t tiles_per = (ntiles + nparts - 1) / nparts;
    const uint32_t part = chunk * (kBwdThreads / 32) + warp;
    const uint32_t begin = min(part * tiles_per, ntiles) * kTile;
    const uint32_t end = min(min((part + 1) * tiles_per, ntiles) * kTile, V);
    float* out = p.d_logits + row * V;

    const float glp = p.g_logp ? p.g_logp[row] : 0.f;
    const float gkl = (REF && p.g_kl) ? p.g_kl[row] : 0.f;
    const float gen = p.g_ent ? p.g_ent[row] : 0.f;
    if (glp == 0.f && gkl == 0.f && gen == 0.f) {
        // an unscored position: exact zeros, the inputs are not read
        for (uint32_t t = begin; t < end; t += kTile) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t e = t + h * (kTile / 2) + lane * 4;
                if (e < end) stg_stream16(out + e, 0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }
    const float4 st = reinterpret_cast<const float4*>(p.rowstats)[row];
    const float m = st.x, lnZ = st.y, mr = st.z, lnZr = st.w;
    const float klv = (REF && p.kl && gkl != 0.f) ? p.kl[row] : 0.f;
    const float hv = (p.entropy && gen != 0.f) ? p.entropy[row] : 0.f;
    const int32_t tok = (p.tokens && glp != 0.f) ? p.tokens[row] : -1;

    typedef VecLoader<DT, REF, true, false, true> Loader;
    uint32_t* wq = queues[warp];
    uint32_t head = 0, count = 0;  // warp-uniform ring state
    Loader pend;
    uint32_t pend_v = kNoEntry;
    bool pend_any = false;

#if NRL_MASK_BITS
    const uint8_t* mp = f.allow + row * f.allow_stride + ((begin + lane * kVec) >> 3);
    constexpr uint32_t kTileMask = kTile / 8;
#else
    const uint8_t* mp = f.allow + row * f.allow_stride + begin + lane * kVec;
    constexpr uint32_t kTileMask = kTile;
#endif
    uint32_t v = begin + lane * kVec;  // this lane's vector of the tile at t0
    uint32_t t0 = begin;
    uint32_t mk[kBwdAhead];
    MaskAny mn[kBwdAhead];
#pragma unroll
    for (int j = 0; j < kBwdAhead; j++) mk[j] = (v + j * kTile < end) ? mask_any_value(ldg_mask_any(mp + j * kTileMask, 0)) : 0u;

    for (;;) {
        const bool scanning = t0 < end;
        if (scanning) {
            const uint8_t* np = mp + kBwdAhead * kTileMask;
            const uint32_t nv = v + kBwdAhead * kTile;
#pragma unroll
            for (int j = 0; j < kBwdAhead; j++) mn[j] = (nv + j * kTile < end) ? ldg_mask_any(np + j * kTileMask, 0) : mask_any_none();
#pragma unroll
            for (int j = 0; j < kBwdAhead; j++) {
                const uint32_t vv = v + j * kTile;
                // a vector is live when it allows a token, or holds the row's token (whose entry gets g_lp even if excluded)
                const bool nz = vv < end && (mk[j] != 0u || (tok >= (int32_t)vv && tok < (int32_t)(vv + kVec)));
                const uint32_t ball = __ballot_sync(0xffffffffu, nz);
                if (nz) wq[(head + count + __popc(ball & lt)) & (kBwdQueue - 1)] = vv;
                count += __popc(ball);
                // zeros for the excluded vectors of this tile: lane l writes elements 4l.. of each half, which belong to vector 16h + l/2
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t e = t0 + j * kTile + h * (kTile / 2) + lane * 4;
                    if (e < end && !((ball >> (h * 16 + (lane >> 1))) & 1u)) stg_stream16(out + e, 0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int j = 0; j < kBwdAhead; j++) mk[j] = mask_any_value(mn[j]);
            mp = np;
            v = nv;
            t0 += kBwdAhead * kTile;
            __syncwarp();
        }
        while (count >= 32 || (!scanning && (count > 0 || pend_any))) {
            const uint32_t n = count < 32 ? count : 32;
            Loader nxt;
            const uint32_t nv_entry = ((uint32_t)lane < n) ? wq[(head + lane) & (kBwdQueue - 1)] : kNoEntry;
            if (nv_entry != kNoEntry) nxt.load(f, row, nv_entry, end);
            head = (head + n) & (kBwdQueue - 1);
            count -= n;
            if (pend_any && pend_v != kNoEntry) {
                float z[8], zr[8], g[8];
                pend.values(f, z, zr);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float zc = fmaxf(z[i], -FLT_MAX);
                    const float lp = (zc - m) - lnZ;
                    const float pi = ex2_approx(lp * kLog2e);
                    float c = -glp;                                          // d logp / dz_j = 1[j = tok] − π_j
                    if (REF) c = fmaf(gkl, (lp - ((zr[i] - mr) - lnZr)) - klv, c);  // d KL / dz_j = π_j (log π_j − log ρ_j − KL)
                    c = fmaf(-gen, lp + hv, c);                              // d H / dz_j = −π_j (log π_j + H)
                    float d = pi > 0.f ? pi * c : 0.f;                       // a zero-probability token gets exactly 0
                    if ((int32_t)(pend_v + i) == tok) d += glp;
                    g[i] = d;
                }
                stg_stream16(out + pend_v, g[0], g[1], g[2], g[3]);
                stg_stream16(out + pend_v + 4, g[4], g[5], g[6], g[7]);
            }
            pend = nxt;
            pend_v = nv_entry;
            pend_any = n > 0;
        }
        if (!scanning) break;
        __syncwarp();  // the batch's entries are read before the next group's pushes can reuse slots
    }
}

}  // namespace nrl
