// Generic reductions along the last axis ("lanes") of a [rows, V] tensor, block-per-row with
// 64-bit offsets: softmax, log_softmax, logsumexp and their backward rules
// (src/tensor/activation.rs:15-42, 71-77), the first-maximum NaN-propagating argmax
// (src/tensor/kernels.rs:184-209, src/tensor/cuda/kernels.rs:656-670) and the lane sum in the
// reference's own operand order (src/tensor/kernels.rs:122-148, cuda/kernels.rs:602-629), which is
// bit-equal to Cpu(Reference) for f32 input.
//
// The softmax family reads a row twice (the second read is an L2 hit while the rows in flight fit
// L2; longer rows are held in the shared memory of a thread-block cluster instead and read once) and
// writes it once; reductions are butterflies over lanes, then over warps, in a fixed tree, so
// results do not depend on timing.
#pragma once
#include "common.cuh"

namespace nrl {

constexpr int kLaneThreads = 256;       // default block; long rows run 1024-thread blocks, one per SM
constexpr int kLaneMaxThreads = 1024;
constexpr int kLaneMaxWarps = kLaneMaxThreads / 32;

// L2 eviction priorities for the rows the softmax family reads twice: the first read asks L2 to keep
// the lines (evict_last), the second marks them as the first to go (evict_first), so that the rows
// in flight, not the output being written, are what L2 holds.
#ifndef NRL_SOFTMAX_HINT
#define NRL_SOFTMAX_HINT 1
#endif
__device__ __forceinline__ uint64_t l2_policy_keep() {
    uint64_t p;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_drop() {
    uint64_t p;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint4 ldg_hint16(const void* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    return v;
}

// Eight consecutive elements of a row as floats; `n` of them exist. VEC: 16-byte loads (every row
// starts on a 16-byte boundary and V is a multiple of 8).
template <int DT, bool VEC>
__device__ __forceinline__ int lane_load8(const void* base, uint64_t row0, uint32_t v, uint32_t V, float z[8], uint64_t policy = 0) {
    Raw<DT> raw;
    const uint32_t e0 = v * kVec;
    int n = kVec;
    if (VEC) {
        if (NRL_SOFTMAX_HINT && policy) {
            if constexpr (DT == NRL_BF16) {
                raw.q = ldg_hint16((const uint16_t*)base + row0 + e0, policy);
            } else {
                raw.a = ldg_hint16((const float*)base + row0 + e0, policy);
                raw.b = ldg_hint16((const float*)base + row0 + e0 + 4, policy);
            }
        } else {
            raw.load(base, row0 + e0);
        }
    } else {
        n = (int)(V - e0 < (uint32_t)kVec ? V - e0 : (uint32_t)kVec);
        raw.load_scalar(base, row0 + e0, n);
    }
    raw.unpack(z);
    return n;
}

template <bool VEC>
__device__ __forceinline__ void lane_store8(float* out, uint64_t row0, uint32_t v, int n, const float y[8]) {
    float* p = out + row0 + (uint64_t)v * kVec;
    if (VEC) {
        stg_stream16(p, y[0], y[1], y[2], y[3]);
        stg_stream16(p + 4, y[4], y[5], y[6], y[7]);
    } else {
#pragma unroll
        for (int i = 0; i < kVec; i++)
            if (i < n) p[i] = y[i];
    }
}

// A full warp tile (256 consecutive elements) for the kernels that write a [rows, V] result: lane l works on the two
// runs of four elements at 4·l and 128 + 4·l of the tile, so that each of the warp's loads and stores covers consecutive
// bytes. (With eight consecutive elements per lane the two 16-byte stores of an f32 result each fill half of every
// 32-byte sector: measured 1.2 × slower on B200.) `elem0` is the tile's first element in the tensor.
template <int DT>
__device__ __forceinline__ void lane_load4x2(const void* base, uint64_t elem0, int lane, float z[8], uint64_t policy = 0) {
    if constexpr (DT == NRL_BF16) {
        const uint16_t* p = (const uint16_t*)base + elem0 + 4 * lane;
        uint2 a, b;
        if (NRL_SOFTMAX_HINT && policy) {
            asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;" : "=r"(a.x), "=r"(a.y) : "l"(p), "l"(policy));
            asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;" : "=r"(b.x), "=r"(b.y) : "l"(p + 128), "l"(policy));
        } else {
            asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(a.x), "=r"(a.y) : "l"(p));
            asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(b.x), "=r"(b.y) : "l"(p + 128));
        }
        z[0] = bf16_lo(a.x); z[1] = bf16_hi(a.x); z[2] = bf16_lo(a.y); z[3] = bf16_hi(a.y);
        z[4] = bf16_lo(b.x); z[5] = bf16_hi(b.x); z[6] = bf16_lo(b.y); z[7] = bf16_hi(b.y);
    } else {
        const float* p = (const float*)base + elem0 + 4 * lane;
        Raw<NRL_F32> raw;
        if (NRL_SOFTMAX_HINT && policy) {
            raw.a = ldg_hint16(p, policy);
            raw.b = ldg_hint16(p + 128, policy);
        } else {
            raw.a = ldg_stream16(p);
            raw.b = ldg_stream16(p + 128);
        }
        raw.unpack(z);
    }
}
__device__ __forceinline__ void lane_store4x2(float* out, uint64_t elem0, int lane, const float y[8]) {
    float* p = out + elem0 + 4 * lane;
    stg_stream16(p, y[0], y[1], y[2], y[3]);
    stg_stream16(p + 128, y[4], y[5], y[6], y[7]);
}

// ---- block reductions in a fixed order ----------------------------------------------------------
// (max, Σ exp(· − max)) pairs
struct MaxSum {
    float m, S;
};
// A sum at maximum m as a sum at maximum M ≥ m (or NaN). A −inf maximum with a finite M drops the sum (it is 0, or the
// NaN of a part that held only −inf); equal maxima keep it as it is, also when both are −inf.
__device__ __forceinline__ float maxsum_rescale(float m, float S, float M) { return m == M ? S : (m == NRL_NEG_INF ? 0.f : S * expf(m - M)); }

// One warp merges up to 32 (max, Σ exp) pairs, one per lane (lanes without a pair pass (−inf, 0)): the maximum by a
// butterfly, every sum rescaled to it once, the sums by a butterfly. Every lane returns the same bits, whatever the
// timing: the tree is fixed.
__device__ __forceinline__ MaxSum warp_maxsum(MaxSum p) {
    float M = p.m;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) M = fmax_nan(M, __shfl_xor_sync(0xffffffffu, M, s));
    float S = maxsum_rescale(p.m, p.S, M);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) S = __fadd_rn(S, __shfl_xor_sync(0xffffffffu, S, s));
    MaxSum r;
    r.m = M;
    r.S = S;
    return r;
}

// threads -> warps -> block: every warp merges the warps' pairs for itself; every thread returns the same bits
__device__ __forceinline__ MaxSum block_maxsum(MaxSum p, float* sh /* 2 * kLaneMaxWarps */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    p = warp_maxsum(p);
    __syncthreads();  // the previous row's readers of sh are done
    if (lane == 0) { sh[2 * warp] = p.m; sh[2 * warp + 1] = p.S; }
    __syncthreads();
    MaxSum w;
    w.m = lane < nwarps ? sh[2 * lane] : NRL_NEG_INF;
    w.S = lane < nwarps ? sh[2 * lane + 1] : 0.f;
    return warp_maxsum(w);
}

__device__ __forceinline__ float block_sum(float x, float* sh /* kLaneMaxWarps */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) x = __fadd_rn(x, __shfl_xor_sync(0xffffffffu, x, s));
    __syncthreads();
    if (lane == 0) sh[warp] = x;
    __syncthreads();
    float r = sh[0];
    const int nwarps = blockDim.x >> 5;
    for (int w = 1; w < nwarps; w++) r = __fadd_rn(r, sh[w]);
    return r;
}

// first maximum, the first NaN being the maximum of a lane that holds one
__device__ __forceinline__ bool arg_better(float e, uint32_t i, float best, uint32_t idx) {
    const bool en = e != e, bn = best != best;
    if (en || bn) return en && (!bn || i < idx);
    return e > best || (e == best && i < idx);
}

// ---- softmax / log_softmax / logsumexp forward -------------------------------------------------
// One thread's (max, Σ exp) over the vectors v = threadIdx.x, threadIdx.x + 256, … of the row.
// Elements beyond V read as −inf. While the running maximum is still −inf the sum is NaN
// (−inf − −inf); the first finite element resets it, so a lane of −inf alone ends as NaN, as the
// reference's (x − max).exp() does.
template <int DT, bool VEC>
__device__ __forceinline__ MaxSum lane_thread_maxsum(const void* x, uint64_t row0, uint32_t V, uint32_t nvec, uint64_t policy = 0) {
    MaxSum p;
    p.m = NRL_NEG_INF;
    p.S = 0.f;
#pragma unroll 2
    for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float z[8];
        lane_load8<DT, VEC>(x, row0, v, V, z, policy);
        const float vmax = fmax_nan(fmax3_nan(z[0], z[1], z[2]), fmax_nan(fmax3_nan(z[3], z[4], z[5]), fmax_nan(z[6], z[7])));
        const float mn = fmax_nan(p.m, vmax);
        if (mn != p.m) {
            p.S = (p.m == NRL_NEG_INF) ? 0.f : p.S * expf(p.m - mn);
            p.m = mn;
        }
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; i++) e[i] = ex2_approx((z[i] - p.m) * kLog2e);
        p.S += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
    }
    return p;
}

template <int DT, bool VEC, bool LOG>
__global__ void __launch_bounds__(kLaneMaxThreads) lane_softmax_kernel(const void* __restrict__ x, float* __restrict__ out, uint64_t rows, uint32_t V) {
    __shared__ float sh[2 * kLaneMaxWarps];
    const uint32_t nvec = (V + kVec - 1) / kVec;
    const uint64_t keep = l2_policy_keep(), drop = l2_policy_drop();
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint64_t row0 = row * V;
        const MaxSum p = block_maxsum(lane_thread_maxsum<DT, VEC>(x, row0, V, nvec, keep), sh);
        const float m = p.m, lnS = logf(p.S), inv = 1.f / p.S;
#pragma unroll 2
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float z[8], y[8];
            const int lane = threadIdx.x & 31;
            const bool tile = VEC && DT == NRL_F32 && (v - lane) + 32 <= nvec;  // the warp holds a full tile (bf16 rows keep their 16-byte loads: measured)
            int n = kVec;
            if (tile) lane_load4x2<DT>(x, row0 + (uint64_t)(v - lane) * kVec, lane, z, drop);
            else n = lane_load8<DT, VEC>(x, row0, v, V, z, drop);
#pragma unroll
            for (int i = 0; i < 8; i++) y[i] = LOG ? (z[i] - m) - lnS : ex2_approx((z[i] - m) * kLog2e) * inv;
            if (tile) lane_store4x2(out, row0 + (uint64_t)(v - lane) * kVec, lane, y);
            else lane_store8<VEC>(out, row0, v, n, y);
        }
    }
}

// ---- softmax / log_softmax of long rows: the row held in a cluster's shared memory ------------------
// A row too long for L2 to keep until its second read (1184 rows of 128 256 f32 are in flight in the
// kernel above: 0.6 GB) is read from HBM twice there: 12 bytes per f32 element for 8 of results and
// operands. Here a thread-block cluster owns a row: each of its CTAs copies one slice of the row into
// its shared memory (cp.async, the whole slice in flight at once), folds the slice into a (max, Σ exp)
// pair, sends the pair into every CTA's shared memory (st.async onto the receiver's mbarrier: unlike a
// cluster barrier it does not wait for the sender's global stores in flight), merges the cluster's
// pairs by a fixed tree (the same bits in every CTA) and writes its slice's results from shared memory.
// The row crosses HBM once in each direction. The exchange slots and mbarriers alternate with the
// row's parity: a CTA can be sent row r + 2's pairs only after it has sent its own pair of row r + 1,
// which it does after it has read row r's.
constexpr int kLaneClusterThreads = 256;  // 512 measured slower
constexpr unsigned long long kLaneWaitLimitNs = 2000000000ull;  // a CTA waits this long for its cluster's pairs
constexpr uint32_t kLaneSliceBytes = 74 * 1024;      // a CTA's slice: three CTAs per SM
constexpr uint32_t kLaneSliceBytesTwo = 112 * 1024;  // or, for rows that need it, two
constexpr uint32_t kLaneMaxCluster = 8;          // the portable cluster size (clusters of 10 to 16 measured slower)

// four consecutive elements of a slice in shared memory: piece q
template <int DT>
__device__ __forceinline__ void lane_piece4(uint32_t slice, uint32_t q, float z[4]) {
    if constexpr (DT == NRL_BF16) {
        uint2 w;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w.x), "=r"(w.y) : "r"(slice + q * 8u));
        z[0] = bf16_lo(w.x); z[1] = bf16_hi(w.x); z[2] = bf16_lo(w.y); z[3] = bf16_hi(w.y);
    } else {
        const uint4 w = lds16(slice + q * 16u);
        z[0] = __uint_as_float(w.x); z[1] = __uint_as_float(w.y); z[2] = __uint_as_float(w.z); z[3] = __uint_as_float(w.w);
    }
}

// (The backward of log_softmax was tried on the same scheme, the upstream gradient held by the cluster: at 148 rows in
// flight L2 already serves the kernel below its second read of g, and the cluster form was 10 % slower.)
template <int DT, bool LOG>
__global__ void __launch_bounds__(kLaneClusterThreads) lane_softmax_cluster_kernel(const void* __restrict__ x, float* __restrict__ out, uint64_t rows, uint32_t V, uint32_t per) {
    extern __shared__ __align__(16) unsigned char lane_slice[];
    __shared__ __align__(8) float2 warp_pair[kLaneClusterThreads / 32];
    __shared__ __align__(8) float2 exchange[2][kLaneMaxCluster];
    __shared__ __align__(8) uint64_t arrived[2];
    constexpr uint32_t kVecBytes = kVec * (DT == NRL_F32 ? 4u : 2u);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint32_t rank = cluster_cta_rank(), csize = cluster_cta_count();
    const uint64_t cluster = blockIdx.x / csize, nclusters = gridDim.x / csize;
    const uint32_t nvec = V / kVec;  // the caller sends rows of whole, 16-byte aligned vectors only
    const uint32_t v0 = rank * per < nvec ? rank * per : nvec;
    const uint32_t n = nvec - v0 < per ? nvec - v0 : per;  // this CTA's vectors: v0 .. v0 + n
    const uint32_t slice = smem_addr(lane_slice), copies = n * (kVecBytes / 16u), pieces = 2 * n;
    // (Copying the next row's slice into a second buffer meanwhile was measured too: the cluster must then be twice
    // as large for the same shared memory, and larger clusters were slower than what the overlap gained.)
    auto fetch = [&](uint64_t row) {
        if (row < rows) {
            const unsigned char* src = (const unsigned char*)x + (row * V + (uint64_t)v0 * kVec) * (kVecBytes / kVec);
            for (uint32_t i = threadIdx.x; i < copies; i += blockDim.x) cp_async16(slice + i * 16u, src + (uint64_t)i * 16u);
        }
        cp_async_commit();
    };
    fetch(cluster);
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&arrived[0]), 1);
        mbar_init(smem_addr(&arrived[1]), 1);
        mbar_init_fence();
    }
    cluster_sync_all();  // no pair is sent to a CTA whose mbarriers are not set up yet
    uint32_t parity = 0, phase = 0;
    bool failed = false;
    for (uint64_t row = cluster; row < rows; row += nclusters, parity ^= 1u) {
        cp_async_wait<0>();
        __syncthreads();  // the row's slice is complete, and everyone is done with the previous row
        // this thread's pieces q, q + blockDim (consecutive lanes read consecutive pieces: no bank conflicts), two per step
        MaxSum p;
        p.m = NRL_NEG_INF;
        p.S = 0.f;
        for (uint32_t q = threadIdx.x; q < pieces; q += 2 * blockDim.x) {
            float z[8];
            lane_piece4<DT>(slice, q, z);
            if (q + blockDim.x < pieces) {
                lane_piece4<DT>(slice, q + blockDim.x, z + 4);
            } else {
                z[4] = z[5] = z[6] = z[7] = NRL_NEG_INF;
            }
            const float vmax = fmax_nan(fmax3_nan(z[0], z[1], z[2]), fmax_nan(fmax3_nan(z[3], z[4], z[5]), fmax_nan(z[6], z[7])));
            const float mn = fmax_nan(p.m, vmax);
            if (mn != p.m) {
                p.S = (p.m == NRL_NEG_INF) ? 0.f : p.S * expf(p.m - mn);
                p.m = mn;
            }
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = ex2_approx((z[i] - p.m) * kLog2e);
            p.S += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
        }
        // threads -> warp -> CTA: every warp merges the warps' pairs for itself, so one barrier is enough
        p = warp_maxsum(p);
        if (lane == 0) warp_pair[warp] = make_float2(p.m, p.S);
        __syncthreads();
        {
            const float2 w = lane < nwarps ? warp_pair[lane] : make_float2(NRL_NEG_INF, 0.f);
            p.m = w.x;
            p.S = w.y;
            p = warp_maxsum(p);
        }
        // CTA -> cluster: every CTA sends its pair to every CTA (itself included) and waits for the cluster's
        // pairs on its own mbarrier. The wait is bounded: a CTA that gives up writes NaN rows from then on.
        MaxSum t;
        t.m = t.S = __int_as_float(0x7fc00000);
        if (!failed) {
            const uint32_t bar = smem_addr(&arrived[parity]);
            if (threadIdx.x == 0) mbar_expect_tx(bar, csize * (uint32_t)sizeof(float2));
            if (threadIdx.x < csize) st_async_f2(in_cluster_cta(smem_addr(&exchange[parity][rank]), threadIdx.x), p.m, p.S, in_cluster_cta(bar, threadIdx.x));
            bool done = mbar_try_wait(bar, phase);
            if (!done) {
                const unsigned long long t0 = global_ns();
                for (uint32_t i = 1; !(done = mbar_try_wait(bar, phase)); i++)
                    if ((i & 63u) == 0u && global_ns() - t0 > kLaneWaitLimitNs) break;
            }
            done = __all_sync(0xffffffffu, done);
            if (done) {
                const float2 c = lane < csize ? exchange[parity][lane] : make_float2(NRL_NEG_INF, 0.f);
                t.m = c.x;
                t.S = c.y;
                t = warp_maxsum(t);
            } else {
                failed = true;
            }
        }
        phase ^= parity;  // each mbarrier is used every second row
        // four elements per thread and step: a warp's store covers 512 consecutive bytes (with eight, its two
        // 16-byte stores would each fill half of every 32-byte sector)
        float* dst = out + row * V + (uint64_t)v0 * kVec;
        const float m = t.m, lnS = logf(t.S), inv = 1.f / t.S;
        // f32 rows: as soon as a piece has been read for the last time, the same thread requests the next row's 16
        // bytes for that place, so the copy of row r + 1 is in flight while row r is still being written (+4 %). A
        // 16-byte copy is two bf16 pieces, read by two lanes; pairing them up cost more than it gained: bf16 rows
        // request the next slice after the pass.
        constexpr bool kEarly = DT == NRL_F32;
        const bool more = row + nclusters < rows;
        const unsigned char* next = (const unsigned char*)x + ((row + nclusters) * V + (uint64_t)v0 * kVec) * (kVecBytes / kVec);
#pragma unroll 4
        for (uint32_t q = threadIdx.x; q < pieces; q += blockDim.x) {
            float z[4], y[4];
            lane_piece4<DT>(slice, q, z);
            if (kEarly && more) cp_async16(slice + q * 16u, next + (uint64_t)q * 16u);
#pragma unroll
            for (int i = 0; i < 4; i++) y[i] = LOG ? (z[i] - m) - lnS : ex2_approx((z[i] - m) * kLog2e) * inv;
            stg_stream16(dst + (uint64_t)q * 4, y[0], y[1], y[2], y[3]);
        }
        if constexpr (kEarly) {
            cp_async_commit();
        } else {
            __syncthreads();  // the slice is free for the next row
            fetch(row + nclusters);
        }
    }
    cluster_sync_all();  // no CTA leaves while a peer may still send to it
}

// m + log Σ exp(x − m), the shift dropped where m is ±inf (a lane of −inf gives −inf, one holding
// +inf gives +inf); NaN propagates through the maximum.
template <int DT, bool VEC>
__global__ void __launch_bounds__(kLaneMaxThreads) lane_logsumexp_kernel(const void* __restrict__ x, float* __restrict__ out, uint64_t rows, uint32_t V) {
    __shared__ float sh[2 * kLaneMaxWarps];
    const uint32_t nvec = (V + kVec - 1) / kVec;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const MaxSum p = block_maxsum(lane_thread_maxsum<DT, VEC>(x, row * V, V, nvec), sh);
        if (threadIdx.x == 0) {
            const float inf = __int_as_float(0x7f800000);
            out[row] = (p.m == inf) ? inf : (p.m == -inf ? -inf : p.m + logf(p.S));
        }
    }
}

// dx = g[row] · exp(x − out[row])
template <int DT, bool VEC>
__global__ void __launch_bounds__(kLaneMaxThreads) lane_logsumexp_bwd_kernel(const void* __restrict__ x, const float* __restrict__ lse, const float* __restrict__ g,
                                                                          float* __restrict__ dx, uint64_t rows, uint32_t V) {
    const uint32_t nvec = (V + kVec - 1) / kVec;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float o = __ldg(lse + row), gr = __ldg(g + row);
#pragma unroll 2
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float z[8], y[8];
            const int lane = threadIdx.x & 31;
            const bool tile = VEC && (v - lane) + 32 <= nvec;
            int n = kVec;
            if (tile) lane_load4x2<DT>(x, row * V + (uint64_t)(v - lane) * kVec, lane, z);
            else n = lane_load8<DT, VEC>(x, row * V, v, V, z);
#pragma unroll
            for (int i = 0; i < 8; i++) y[i] = gr * ex2_approx((z[i] - o) * kLog2e);
            if (tile) lane_store4x2(dx, row * V + (uint64_t)(v - lane) * kVec, lane, y);
            else lane_store8<VEC>(dx, row * V, v, n, y);
        }
    }
}

// softmax: dx = y · (g − Σ g·y);  log_softmax: dx = g − exp(y) · Σ g   (y the saved output, f32)
template <bool VEC, bool LOG>
__global__ void __launch_bounds__(kLaneMaxThreads) lane_softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ g, float* __restrict__ dx,
                                                                        uint64_t rows, uint32_t V) {
    __shared__ float sh[kLaneMaxWarps];
    const uint32_t nvec = (V + kVec - 1) / kVec;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint64_t row0 = row * V;
        float acc = 0.f;
#pragma unroll 2
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float a[8], b[8], t[8];
            const int n = lane_load8<NRL_F32, VEC>(g, row0, v, V, a);
            if (!LOG) lane_load8<NRL_F32, VEC>(y, row0, v, V, b);
#pragma unroll
            for (int i = 0; i < 8; i++) t[i] = (i < n) ? (LOG ? a[i] : a[i] * b[i]) : 0.f;
            acc += ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
        }
        const float s = block_sum(acc, sh);
#pragma unroll 2
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float a[8], b[8], d[8];
            const int lane = threadIdx.x & 31;
            const bool tile = VEC && (v - lane) + 32 <= nvec;
            int n = kVec;
            if (tile) {
                lane_load4x2<NRL_F32>(g, row0 + (uint64_t)(v - lane) * kVec, lane, a);
                lane_load4x2<NRL_F32>(y, row0 + (uint64_t)(v - lane) * kVec, lane, b);
            } else {
                n = lane_load8<NRL_F32, VEC>(g, row0, v, V, a);
                lane_load8<NRL_F32, VEC>(y, row0, v, V, b);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) d[i] = LOG ? a[i] - ex2_approx(b[i] * kLog2e) * s : b[i] * (a[i] - s);
            if (tile) lane_store4x2(dx, row0 + (uint64_t)(v - lane) * kVec, lane, d);
            else lane_store8<VEC>(dx, row0, v, n, d);
        }
    }
}

// ---- argmax -------------------------------------------------------------------------------------
template <int DT, bool VEC>
__global__ void __launch_bounds__(kLaneMaxThreads) lane_argmax_kernel(const void* __restrict__ x, int32_t* __restrict__ out_index, float* __restrict__ out_value,
                                                                   uint64_t rows, uint32_t V) {
    __shared__ float shv[kLaneMaxWarps];
    __shared__ uint32_t shi[kLaneMaxWarps];
    const uint32_t nvec = (V + kVec - 1) / kVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float best = NRL_NEG_INF;
        uint32_t idx = 0xffffffffu;  // "nothing seen": any element of the row beats it, also a −inf one
#pragma unroll 2
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            float z[8];
            const int n = lane_load8<DT, VEC>(x, row * V, v, V, z);
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i < n && arg_better(z[i], v * kVec + i, best, idx)) { best = z[i]; idx = v * kVec + i; }
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, s);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, s);
            if (arg_better(ob, oi, best, idx)) { best = ob; idx = oi; }
        }
        __syncthreads();
        if (lane == 0) { shv[warp] = best; shi[warp] = idx; }
        __syncthreads();
        if (threadIdx.x == 0) {
            best = shv[0]; idx = shi[0];
            for (int w = 1; w < (int)(blockDim.x >> 5); w++)
                if (arg_better(shv[w], shi[w], best, idx)) { best = shv[w]; idx = shi[w]; }
            out_index[row] = (int32_t)idx;
            if (out_value) out_value[row] = best;
        }
    }
}

// ---- the lane sum in the reference's operand order ---------------------------------------------
// Eight partial sums p_k = x[k] + x[8 + k] + x[16 + k] + …, each built left to right, combined as
// acc = 0; acc += p0 + p4; acc += p1 + p5; acc += p2 + p6; acc += p3 + p7; then the V mod 8 tail in
// order. Eight lanes own a row (one partial each), so a warp streams four rows and every load
// instruction reads four whole 32-byte sectors; the adds of one partial are dependent by
// definition, the loads are issued 32 deep ahead of them.
template <int DT>
__device__ __forceinline__ float lane_elem(const void* x, uint64_t i) {
    if (DT == NRL_BF16) return __uint_as_float((uint32_t)__ldg((const uint16_t*)x + i) << 16);
    return __ldg((const float*)x + i);
}

template <int DT>
__global__ void __launch_bounds__(kLaneThreads) lane_sum_ordered_kernel(const void* __restrict__ x, float* __restrict__ out, uint64_t rows, uint32_t V) {
    const int k = threadIdx.x & 7;
    const uint64_t rows_per_block = blockDim.x / 8;
    const uint32_t full = V / 8;
    for (uint64_t base = (uint64_t)blockIdx.x * rows_per_block; base < rows; base += (uint64_t)gridDim.x * rows_per_block) {
        const uint64_t row = base + (threadIdx.x >> 3);
        const bool live = row < rows;  // every lane stays for the shuffles
        const uint64_t row0 = (live ? row : 0) * V;
        float p = 0.f;
        uint32_t j = 0;
        if (live) {
            // Two batches of kSumDepth loads: the next batch is issued before the current one is added, so
            // loads are in flight during the dependent adds too (eight threads per row leave an SM few
            // warps; what hides the latency is the depth per thread).
            constexpr int kSumDepth = 48;
            float t[2][kSumDepth];
            const uint32_t nb = full / kSumDepth;  // whole batches
            auto load = [&](float* dst, uint32_t b) {
#pragma unroll
                for (int u = 0; u < kSumDepth; u++) dst[u] = lane_elem<DT>(x, row0 + (uint64_t)(b * kSumDepth + u) * 8 + k);
            };
            auto add = [&](const float* src) {
#pragma unroll
                for (int u = 0; u < kSumDepth; u++) p = __fadd_rn(p, src[u]);
            };
            if (nb > 0) load(t[0], 0);
            for (uint32_t b = 0; b < nb; b += 2) {
                if (b + 1 < nb) load(t[1], b + 1);
                add(t[0]);
                if (b + 1 < nb) {
                    if (b + 2 < nb) load(t[0], b + 2);
                    add(t[1]);
                }
            }
            j = nb * kSumDepth;
            for (; j < full; j++) p = __fadd_rn(p, lane_elem<DT>(x, row0 + (uint64_t)j * 8 + k));
        }
        const float q = __fadd_rn(p, __shfl_down_sync(0xffffffffu, p, 4, 8));  // lanes 0..3 of the row: p_k + p_{k+4}
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, q, i, 8));
        if (live && k == 0) {
            for (uint32_t e = full * 8; e < V; e++) acc = __fadd_rn(acc, lane_elem<DT>(x, row0 + e));
            out[row] = acc;
        }
    }
}

}  // namespace nrl
