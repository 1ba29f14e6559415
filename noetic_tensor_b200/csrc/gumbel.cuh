// The reference's own sampler on the device: Gumbel-max with one ChaCha20 `next_u64` per logit
// (src/nn/rl.rs:490-529). The reference draws the noise on the host, one u64 per logit in
// row-major order, and uploads rows·V floats; here every thread regenerates the keystream words
// of its own logits (ChaCha20 is counter-based: word w of the stream is word w mod 16 of block
// w / 16), so the tokens are those the reference draws from the same seed and stream position.
//
//   k = next_u64() >> 11;  u = (k + ½) / 2^53;  g = (f32)(−ln(−ln u))   (noise in f64, src/nn/rl.rs:490-497)
//   token = first maximum of  z_v + g_v  in f32, z = logits / τ + mask   (src/nn/rl.rs:510-529)
//
// The kernel is bound by integer and f64 arithmetic (one ChaCha20 block and sixteen f64
// logarithms per eight logits that can win), not by memory; vectors a byte mask excludes are skipped.
#pragma once
#include "row_fwd.cuh"

namespace nrl {

struct GumbelParams {
    FwdParams in;          // logits, masks, V, rows, tau
    uint32_t key[8];       // the 32-byte seed as little-endian words
    uint64_t word_offset;  // 32-bit words of the stream already consumed
    int32_t* tokens;
    uint8_t* status;
};

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int n) { return __funnelshift_l(x, x, n); }

#define NRL_QR(a, b, c, d)                       \
    a += b; d ^= a; d = rotl32(d, 16);           \
    c += d; b ^= c; b = rotl32(b, 12);           \
    a += b; d ^= a; d = rotl32(d, 8);            \
    c += d; b ^= c; b = rotl32(b, 7);

// ChaCha20 block `counter` (64-bit block counter, zero stream id) of the key: RFC 8439's block
// function with the counter in words 12-13, as rand_chacha's ChaCha20Rng lays it out.
__device__ __forceinline__ void chacha20_block(const uint32_t* key, uint64_t counter, uint32_t out[16]) {
    const uint32_t c0 = 0x61707865u, c1 = 0x3320646eu, c2 = 0x79622d32u, c3 = 0x6b206574u;
    const uint32_t n0 = (uint32_t)counter, n1 = (uint32_t)(counter >> 32);
    uint32_t x0 = c0, x1 = c1, x2 = c2, x3 = c3, x4 = key[0], x5 = key[1], x6 = key[2], x7 = key[3];
    uint32_t x8 = key[4], x9 = key[5], x10 = key[6], x11 = key[7], x12 = n0, x13 = n1, x14 = 0u, x15 = 0u;
#pragma unroll 2
    for (int r = 0; r < 10; r++) {
        NRL_QR(x0, x4, x8, x12) NRL_QR(x1, x5, x9, x13) NRL_QR(x2, x6, x10, x14) NRL_QR(x3, x7, x11, x15)
        NRL_QR(x0, x5, x10, x15) NRL_QR(x1, x6, x11, x12) NRL_QR(x2, x7, x8, x13) NRL_QR(x3, x4, x9, x14)
    }
    out[0] = x0 + c0; out[1] = x1 + c1; out[2] = x2 + c2; out[3] = x3 + c3;
    out[4] = x4 + key[0]; out[5] = x5 + key[1]; out[6] = x6 + key[2]; out[7] = x7 + key[3];
    out[8] = x8 + key[4]; out[9] = x9 + key[5]; out[10] = x10 + key[6]; out[11] = x11 + key[7];
    out[12] = x12 + n0; out[13] = x13 + n1; out[14] = x14; out[15] = x15;
}
#undef NRL_QR

__device__ __forceinline__ float gumbel_noise(uint32_t lo, uint32_t hi) {
    const uint64_t k = (((uint64_t)hi << 32) | (uint64_t)lo) >> 11;
    const double u = ((double)k + 0.5) * (1.0 / 9007199254740992.0);  // a power of two: the product is the quotient
    return (float)(-log(-log(u)));
}

constexpr int kGumbelThreads = 256;

template <int DT, bool ALLOW, bool VEC>
__global__ void __launch_bounds__(kGumbelThreads) gumbel_argmax_kernel(GumbelParams p) {
    __shared__ float s_best[kGumbelThreads / 32], s_top[kGumbelThreads / 32];
    __shared__ uint32_t s_idx[kGumbelThreads / 32];
    __shared__ uint32_t s_list[ALLOW && VEC ? kGumbelThreads / 32 : 1][ALLOW && VEC ? 16 * 32 : 1];  // a warp's live vectors of one round
    const FwdParams& f = p.in;
    const uint64_t row = blockIdx.x;
    const uint32_t V = f.V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float best = NRL_NEG_INF, top = NRL_NEG_INF;  // best noisy value; maximum of the noise-free logits (NaN-propagating)
    uint32_t bidx = 0xffffffffu;
    VecLoader<DT, false, ALLOW, true, VEC> ld;
    auto fold = [&](uint32_t v) {
        ld.load(f, row, v, V);
        float z[8], zr[8];
        ld.values(f, z, zr);
        // the sixteen stream words of these eight logits: one block when they start on a block boundary
        const uint64_t w = p.word_offset + 2ull * (row * (uint64_t)V + v);
        const uint32_t off = (uint32_t)(w & 15u);
        auto consider = [&](int i, uint32_t lo, uint32_t hi) {
            if (v + i < V) {
                float x = z[i];
                if (ALLOW && x == -FLT_MAX) return;  // a token the byte mask excludes: −inf plus any noise never wins
                top = fmax_nan(top, x);
                const float y = x + gumbel_noise(lo, hi);
                if (y > best || (y == best && v + (uint32_t)i < bidx)) {  // the first maximum stays
                    best = y;
                    bidx = v + i;
                }
            }
        };
        if (off == 0u) {  // the usual case (V and the stream position multiples of 8 logits): registers only
            uint32_t ks[16];
            chacha20_block(p.key, w >> 4, ks);
#pragma unroll
            for (int i = 0; i < 8; i++) consider(i, ks[2 * i], ks[2 * i + 1]);
        } else {
            uint32_t ks[32];
            chacha20_block(p.key, w >> 4, ks);
            chacha20_block(p.key, (w >> 4) + 1ull, ks + 16);
#pragma unroll
            for (int i = 0; i < 8; i++) consider(i, ks[off + 2 * i], ks[off + 2 * i + 1]);
        }
    };
    if constexpr (ALLOW && VEC) {
        // A vector the byte mask excludes cannot win and cannot raise `top`: its keystream block and its sixteen
        // logarithms are not computed. Round by round a warp collects the liveness of its next 16 × 32 vectors
        // (independent 8-byte mask loads), lists the live ones in shared memory and deals them out to its lanes one by
        // one: every lane has a live vector at the arithmetic, instead of one or two lanes per step having work
        // (grammar masks allow a few per cent of the vocabulary) or lanes with few live vectors waiting for lanes with
        // many. A lane no longer sees its vectors in index order; ties are decided by the index.
        const uint8_t* mrow = f.allow + row * f.allow_stride;
        constexpr uint32_t kStride = kGumbelThreads * kVec, kRound = 16;
        uint32_t* list = s_list[warp];
        for (uint32_t base0 = (uint32_t)warp * 32u * kVec; base0 < V; base0 += kRound * kStride) {  // warp-uniform
            const uint32_t base = base0 + (uint32_t)lane * kVec;
            uint32_t live = 0;
#pragma unroll
            for (uint32_t k = 0; k < kRound; k++) {
                const uint32_t v = base + k * kStride;
                if (v < V) {
                    const uint2 q = ldg_mask8(mrow, v);
                    live |= (uint32_t)((q.x | q.y) != 0u) << k;
                }
            }
            uint32_t incl = (uint32_t)__popc(live);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
            uint32_t pos = incl - (uint32_t)__popc(live);
            while (live) {
                const uint32_t k = (uint32_t)__ffs((int)live) - 1u;
                live &= live - 1u;
                list[pos++] = base + k * kStride;
            }
            __syncwarp();
            for (uint32_t e = (uint32_t)lane; e < total; e += 32u) fold(list[e]);
            __syncwarp();  // the list is read before the next round rewrites it
        }
    } else {
        for (uint32_t v = threadIdx.x * kVec; v < V; v += kGumbelThreads * kVec) fold(v);
    }
    // the block's first maximum: larger value, then smaller index
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, s);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bidx, s);
        top = fmax_nan(top, __shfl_xor_sync(0xffffffffu, top, s));
        if (ob > best || (ob == best && oi < bidx)) {
            best = ob;
            bidx = oi;
        }
    }
    if (lane == 0) {
        s_best[warp] = best;
        s_idx[warp] = bidx;
        s_top[warp] = top;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < kGumbelThreads / 32; k++) {
            top = fmax_nan(top, s_top[k]);
            if (s_best[k] > best || (s_best[k] == best && s_idx[k] < bidx)) {
                best = s_best[k];
                bidx = s_idx[k];
            }
        }
        uint32_t status = 0;
        if (top != top) status = 2u;                  // a NaN
        else if (top == NRL_NEG_INF) status = 1u;     // no allowed token
        p.tokens[row] = status ? -1 : (int32_t)bidx;
        if (p.status) p.status[row] = (uint8_t)status;
    }
}

}  // namespace nrl
