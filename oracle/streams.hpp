// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// The random streams and 16-bit float conversions the reference's `nn::rl` path depends on,
// restated from their published definitions:
//   * SHA-256 (FIPS 180-4), used by `rng::derive` (src/rng.rs:10-17): seed = sha256(root_le ‖ label).
//   * ChaCha20 with a 64-bit block counter in words 12-13 and a zero stream id in words 14-15
//     (the layout of rand_chacha 0.3.1's `ChaCha20Rng`, pinned in the reference's Cargo.lock; its
//     source is not part of the reference tree). Words are consumed in order, block after block;
//     `next_u64` is two consecutive words, low word first (rand_core 0.6.4 `BlockRng`).
//     The reference's tests pin the stream only behaviourally (src/nn/tests/rl.rs:596-615), so
//     the byte stream is checked against RFC 8439's zero-key/zero-nonce keystream instead:
//     PARITY UNPINNED against rand_chacha's own output for this stream (no vector of it exists
//     in the reference tree and the crate cannot be built here).
//   * bfloat16 round-to-nearest-even and exact upcast (src/tensor/half.rs:15-31).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace orc {

struct Sha256 {
    uint32_t h[8];
    uint8_t buf[64];
    uint64_t len = 0;
    size_t fill = 0;
    Sha256() {
        static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
        std::memcpy(h, init, sizeof h);
    }
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74,
            0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d,
            0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e,
            0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5,
            0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
            uint32_t ch = (e & f) ^ (~e & g);
            uint32_t t1 = hh + S1 + ch + K[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
            uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
            uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const void* data, size_t n) {
        const uint8_t* p = (const uint8_t*)data;
        len += n;
        while (n) {
            size_t k = 64 - fill < n ? 64 - fill : n;
            std::memcpy(buf + fill, p, k);
            fill += k; p += k; n -= k;
            if (fill == 64) { block(buf); fill = 0; }
        }
    }
    void finish(uint8_t out[32]) {
        uint64_t bits = len * 8;
        uint8_t pad = 0x80;
        update(&pad, 1);
        uint8_t z = 0;
        while (fill != 56) update(&z, 1);
        uint8_t lb[8];
        for (int i = 0; i < 8; i++) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(lb, 8);
        for (int i = 0; i < 8; i++) {
            out[4 * i] = (uint8_t)(h[i] >> 24); out[4 * i + 1] = (uint8_t)(h[i] >> 16);
            out[4 * i + 2] = (uint8_t)(h[i] >> 8); out[4 * i + 3] = (uint8_t)h[i];
        }
    }
};

struct ChaCha20Rng {
    uint32_t key[8];
    uint64_t counter = 0;
    uint32_t buf[16];
    int idx = 16;

    static uint32_t rotl(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }
    static void qr(uint32_t* s, int a, int b, int c, int d) {
        s[a] += s[b]; s[d] ^= s[a]; s[d] = rotl(s[d], 16);
        s[c] += s[d]; s[b] ^= s[c]; s[b] = rotl(s[b], 12);
        s[a] += s[b]; s[d] ^= s[a]; s[d] = rotl(s[d], 8);
        s[c] += s[d]; s[b] ^= s[c]; s[b] = rotl(s[b], 7);
    }
    static void block_fn(const uint32_t in[16], uint32_t out[16]) {
        uint32_t s[16];
        std::memcpy(s, in, sizeof s);
        for (int r = 0; r < 10; r++) {
            qr(s, 0, 4, 8, 12); qr(s, 1, 5, 9, 13); qr(s, 2, 6, 10, 14); qr(s, 3, 7, 11, 15);
            qr(s, 0, 5, 10, 15); qr(s, 1, 6, 11, 12); qr(s, 2, 7, 8, 13); qr(s, 3, 4, 9, 14);
        }
        for (int i = 0; i < 16; i++) out[i] = s[i] + in[i];
    }
    explicit ChaCha20Rng(const uint8_t seed[32]) {
        for (int i = 0; i < 8; i++) key[i] = (uint32_t)seed[4 * i] | (uint32_t)seed[4 * i + 1] << 8 | (uint32_t)seed[4 * i + 2] << 16 | (uint32_t)seed[4 * i + 3] << 24;
    }
    // src/rng.rs:10-17
    static ChaCha20Rng derive(uint64_t root, const std::string& label) {
        Sha256 h;
        uint8_t le[8];
        for (int i = 0; i < 8; i++) le[i] = (uint8_t)(root >> (8 * i));
        h.update(le, 8);
        h.update(label.data(), label.size());
        uint8_t seed[32];
        h.finish(seed);
        return ChaCha20Rng(seed);
    }
    void refill() {
        uint32_t st[16] = {0x61707865, 0x3320646e, 0x79622d32, 0x6b206574};
        for (int i = 0; i < 8; i++) st[4 + i] = key[i];
        st[12] = (uint32_t)counter;
        st[13] = (uint32_t)(counter >> 32);
        st[14] = 0;
        st[15] = 0;
        block_fn(st, buf);
        counter++;
        idx = 0;
    }
    uint32_t next_u32() {
        if (idx >= 16) refill();
        return buf[idx++];
    }
    uint64_t next_u64() {
        uint64_t lo = next_u32();
        uint64_t hi = next_u32();
        return hi << 32 | lo;
    }
};

// src/tensor/half.rs:15-31
inline uint16_t bf16_from_f32(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    if (x != x) return (uint16_t)((b >> 16) | 0x0040);
    uint32_t round = 0x7fff + ((b >> 16) & 1);
    return (uint16_t)((b + round) >> 16);
}
inline float bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float x;
    std::memcpy(&x, &b, 4);
    return x;
}

}  // namespace orc
