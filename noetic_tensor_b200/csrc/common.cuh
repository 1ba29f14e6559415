// Shared device helpers of the nrl kernels (sm_100a): 128-bit streaming loads, bf16 unpacking,
// NaN-propagating maxima, the exponential used in the streaming loops and the online-softmax
// partial that every level of the fixed reduction tree merges.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <float.h>
#include <math.h>

#include "../../include/nrl.h"

namespace nrl {

#ifndef NRL_THREADS
#define NRL_THREADS 256
#endif
constexpr int kThreads = NRL_THREADS;      // threads per block of the row kernels
constexpr int kWarps = kThreads / 32;      // 16 warps: each owns a contiguous part of the row
constexpr int kVec = 8;                    // elements per thread per step (16 B of bf16)
constexpr int kTile = 32 * kVec;           // elements one warp covers per step
constexpr int kPartFloats = 8;             // floats per stored partial (m, S, W, D, mr, Sr, amax index, pad)
constexpr float kLog2e = 1.4426950408889634f;
#define NRL_NEG_INF (-__int_as_float(0x7f800000))

// ---- loads that bypass L1 allocation: every input byte is read once ----------------------------
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ---- asynchronous global→shared copies (16 bytes per lane, no registers held while in flight) ---
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// ---- mbarriers in shared memory -----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- thread-block clusters ------------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_cta_count() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// `addr` (a shared-memory address of this CTA) as the address of the same offset in the cluster's CTA `rank`
__device__ __forceinline__ uint32_t in_cluster_cta(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
// Two floats into another CTA's shared memory; the 8 bytes count on that CTA's mbarrier when they land. Unlike a
// cluster barrier this orders nothing else: the sender's global stores in flight are not waited for.
__device__ __forceinline__ void st_async_f2(uint32_t remote_addr, float a, float b, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(remote_addr), "f"(a), "f"(b), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// streaming (evict-first) 16-byte store for gradients that are written once and not re-read here
__device__ __forceinline__ void stg_stream16(void* p, float a, float b, float c, float d) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// max that returns NaN if either input is NaN (the reference's maxima propagate NaN,
// src/tensor/kernels.rs:184-209)
__device__ __forceinline__ float fmax_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// three-input NaN-propagating max (one instruction on sm_100)
__device__ __forceinline__ float fmax3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- packed pairs of f32 (sm_100 f32x2 arithmetic: one issue slot for two lanes of work) -------
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x, hardware approximation (relative error about 2^-22)
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ---- the raw 8-element vector of one input stream ----------------------------------------------
template <int DT>
struct Raw;
template <>
struct Raw<NRL_BF16> {
    uint4 q;
    __device__ __forceinline__ void load(const void* base, uint64_t elem) { q = ldg_stream16((const uint16_t*)base + elem); }
    __device__ __forceinline__ void load_scalar(const void* base, uint64_t elem, int n) {
        const uint16_t* p = (const uint16_t*)base + elem;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t lo = (2 * i < n) ? (uint32_t)__ldg(p + 2 * i) : 0xff80u;
            uint32_t hi = (2 * i + 1 < n) ? (uint32_t)__ldg(p + 2 * i + 1) : 0xff80u;
            w[i] = lo | (hi << 16);
        }
        q = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ void unpack(float z[8]) const {
        z[0] = bf16_lo(q.x); z[1] = bf16_hi(q.x); z[2] = bf16_lo(q.y); z[3] = bf16_hi(q.y);
        z[4] = bf16_lo(q.z); z[5] = bf16_hi(q.z); z[6] = bf16_lo(q.w); z[7] = bf16_hi(q.w);
    }
};
template <>
struct Raw<NRL_F32> {
    uint4 a, b;
    __device__ __forceinline__ void load(const void* base, uint64_t elem) {
        a = ldg_stream16((const float*)base + elem);
        b = ldg_stream16((const float*)base + elem + 4);
    }
    __device__ __forceinline__ void load_scalar(const void* base, uint64_t elem, int n) {
        const float* p = (const float*)base + elem;
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = (i < n) ? __float_as_uint(__ldg(p + i)) : 0xff800000u;
        a = make_uint4(w[0], w[1], w[2], w[3]);
        b = make_uint4(w[4], w[5], w[6], w[7]);
    }
    __device__ __forceinline__ void unpack(float z[8]) const {
        z[0] = __uint_as_float(a.x); z[1] = __uint_as_float(a.y); z[2] = __uint_as_float(a.z); z[3] = __uint_as_float(a.w);
        z[4] = __uint_as_float(b.x); z[5] = __uint_as_float(b.y); z[6] = __uint_as_float(b.z); z[7] = __uint_as_float(b.w);
    }
};

// ---- the allow-mask of a row ---------------------------------------------------------------------
// NRL_MASK_BITS 0: a byte per token (`mrow` points at the row's V bytes). NRL_MASK_BITS 1: a bit
// per token (`mrow` points at the row's bit-packed words, read as bytes: bit v of the row is bit
// v mod 8 of byte v / 8, which on a little-endian machine is bit v mod 32 of word v / 32). Either
// way the kernels work on "the eight mask bytes of the vector at element v": with bits they are
// spread out of one byte (0 or 1 each).
#ifndef NRL_MASK_BITS
#define NRL_MASK_BITS 0
#endif
__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t spread4(uint32_t nibble) { return (nibble * 0x00204081u) & 0x01010101u; }  // bit k -> byte k
// the eight mask bytes of the vector at element v (a multiple of 8)
__device__ __forceinline__ uint2 ldg_mask8(const uint8_t* mrow, uint32_t v) {
#if NRL_MASK_BITS
    const uint32_t b = __ldg(mrow + (v >> 3));
    return make_uint2(spread4(b & 0xfu), spread4(b >> 4));
#else
    return ldg_stream8(mrow + v);
#endif
}
// the four mask bytes at element e (a multiple of 4)
__device__ __forceinline__ uint32_t ldg_mask4(const uint8_t* mrow, uint32_t e) {
#if NRL_MASK_BITS
    return spread4((__ldg(mrow + (e >> 3)) >> (e & 4u)) & 0xfu);
#else
    return ldg_stream4(mrow + e);
#endif
}
// what a scan needs of a vector's mask: something that is non-zero iff a token of it is allowed
#if NRL_MASK_BITS
typedef uint32_t MaskAny;
__device__ __forceinline__ MaskAny ldg_mask_any(const uint8_t* mrow, uint32_t v) { return __ldg(mrow + (v >> 3)); }
__device__ __forceinline__ MaskAny mask_any_none() { return 0u; }
__device__ __forceinline__ uint32_t mask_any_value(MaskAny a) { return a; }
#else
typedef uint2 MaskAny;
__device__ __forceinline__ MaskAny ldg_mask_any(const uint8_t* mrow, uint32_t v) { return ldg_stream8(mrow + v); }
__device__ __forceinline__ MaskAny mask_any_none() { return make_uint2(0u, 0u); }
__device__ __forceinline__ uint32_t mask_any_value(MaskAny a) { return a.x | a.y; }
#endif

// eight allow-mask bytes
struct RawMask {
    uint2 q;
    __device__ __forceinline__ void load(const uint8_t* mrow, uint32_t v) { q = ldg_mask8(mrow, v); }
#if NRL_MASK_BITS
    // n tokens from element v on (any v): bits beyond n read as excluded
    __device__ __forceinline__ void load_scalar(const uint8_t* mrow, uint32_t v, int n) {
        uint32_t w = __ldg(mrow + (v >> 3));
        if ((v & 7u) + (uint32_t)n > 8u) w |= (uint32_t)__ldg(mrow + (v >> 3) + 1) << 8;
        w = (w >> (v & 7u)) & ((1u << n) - 1u);
        q = make_uint2(spread4(w & 0xfu), spread4((w >> 4) & 0xfu));
    }
#else
    __device__ __forceinline__ void load_scalar(const uint8_t* mrow, uint32_t v, int n) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (i < n) lo |= (uint32_t)__ldg(mrow + v + i) << (8 * i);
            if (i + 4 < n) hi |= (uint32_t)__ldg(mrow + v + i + 4) << (8 * i);
        }
        q = make_uint2(lo, hi);
    }
#endif
    __device__ __forceinline__ bool allowed(int i) const { return (((i < 4 ? q.x : q.y) >> (8 * (i & 3))) & 0xffu) != 0u; }
    __device__ __forceinline__ bool any() const { return (q.x | q.y) != 0u; }
};

// ---- online-softmax partial ---------------------------------------------------------------------
// Over a set of elements with tempered logits z (policy) and zr (reference):
//   m  = max z,  S = Σ exp(z − m),  W = Σ exp(z − m)·(z − m),  D = Σ exp(z − m)·(z − zr)
//   mr = max zr, Sr = Σ exp(zr − mr)
// An empty set is m = −inf, S = W = D = 0.
struct Partial {
    float m, S, W, D, mr, Sr;
};

__device__ __forceinline__ Partial partial_empty() {
    Partial p;
    p.m = NRL_NEG_INF; p.S = 0.f; p.W = 0.f; p.D = 0.f; p.mr = NRL_NEG_INF; p.Sr = 0.f;
    return p;
}

// Move a partial to a larger (or NaN) maximum `mn`; exact when the maximum does not change.
__device__ __forceinline__ void partial_rebase(float& m, float& S, float& W, float& D, float mn) {
    if (m != mn) {
        if (m == NRL_NEG_INF) {
            S = 0.f; W = 0.f; D = 0.f;
        } else {
            float dm = m - mn;      // ≤ 0, or NaN
            float c = expf(dm);     // accurate: rebasing happens a handful of times per row
            W = c * (W + S * dm);
            S = c * S;
            D = c * D;
        }
        m = mn;
    }
}
__device__ __forceinline__ void partial_rebase_ref(float& mr, float& Sr, float mn) {
    if (mr != mn) {
        Sr = (mr == NRL_NEG_INF) ? 0.f : Sr * expf(mr - mn);
        mr = mn;
    }
}

// a ⊕ b, used at every level of the fixed tree (lanes of a warp, then parts of a row)
__device__ __forceinline__ Partial partial_merge(Partial a, const Partial& b) {
    float mn = fmax_nan(a.m, b.m);
    float bm = b.m, bS = b.S, bW = b.W, bD = b.D;
    partial_rebase(a.m, a.S, a.W, a.D, mn);
    partial_rebase(bm, bS, bW, bD, mn);
    a.S = __fadd_rn(a.S, bS);
    a.W = __fadd_rn(a.W, bW);
    a.D = __fadd_rn(a.D, bD);
    float mrn = fmax_nan(a.mr, b.mr);
    float bmr = b.mr, bSr = b.Sr;
    partial_rebase_ref(a.mr, a.Sr, mrn);
    partial_rebase_ref(bmr, bSr, mrn);
    a.Sr = __fadd_rn(a.Sr, bSr);
    return a;
}

__device__ __forceinline__ Partial partial_shfl_xor(const Partial& p, int mask) {
    Partial o;
    o.m = __shfl_xor_sync(0xffffffffu, p.m, mask);
    o.S = __shfl_xor_sync(0xffffffffu, p.S, mask);
    o.W = __shfl_xor_sync(0xffffffffu, p.W, mask);
    o.D = __shfl_xor_sync(0xffffffffu, p.D, mask);
    o.mr = __shfl_xor_sync(0xffffffffu, p.mr, mask);
    o.Sr = __shfl_xor_sync(0xffffffffu, p.Sr, mask);
    return o;
}

// Butterfly over the 32 lanes in a fixed order; lane 0's result is the one used.
__device__ __forceinline__ Partial partial_warp_reduce(Partial p) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        Partial o = partial_shfl_xor(p, s);
        // the lower lane of each pair merges (own, other) and the upper (other, own): same operands
        // in the same order, so both hold the same bits
        bool low = (threadIdx.x & s) == 0;
        p = low ? partial_merge(p, o) : partial_merge(o, p);
    }
    return p;
}

// inclusive scan of doubles over a warp, lower lanes first
__device__ __forceinline__ double warp_scan_incl(double x, int lane) {
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        double y = __shfl_up_sync(0xffffffffu, x, s);
        if (lane >= s) x = y + x;
    }
    return x;
}

}  // namespace nrl
