// Rows that live in HOST memory, for the byte-masked forward: what crosses PCIe.
//
// The masked forward never reads a logit the mask excludes, so a host caller need not upload
// them. nrl_host_pack (host threads) keeps, per row, one liveness bit per 8-element vector and,
// for the live vectors only, their logits, reference logits and 8 mask bytes, in row order;
// nrl_unpack_rows (a kernel) puts them back at their places in the full [rows, V] device
// buffers and writes the full byte mask (zeros where nothing is allowed). The positions of
// excluded logits in the device buffers are left as they were: nothing reads them.
// With a grammar mask that allows ~5 % of a 128 256-token vocabulary this is 82 KB per row over
// the link instead of 641 KB.
#pragma once
#include <immintrin.h>

#include <unistd.h>

#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace nrl {

// Host threads that stay: the packers below run twice per chunk of a few hundred rows, and starting and joining
// sixteen threads each time cost a fifth of a chunk. One pool per calling thread (thread_local: callers on different
// threads pack at the same time without sharing anything); its workers sleep on a condition variable between runs
// and are joined when the calling thread ends.
class HostPool {
  public:
    ~HostPool() {
        if (getpid() != pid_) return;  // a forked child inherits the object but not the threads: nothing to join
        {
            std::lock_guard<std::mutex> hold(s_->m);
            s_->stop = true;
            s_->gen++;
        }
        s_->start.notify_all();
        for (auto& t : s_->workers) t.join();
        delete s_;
    }
    // fn(t) for t in [0, nt): t = 0 on the calling thread, the rest on workers; returns when all are done
    void run(uint32_t nt, const std::function<void(uint32_t)>& fn) {
        if (nt <= 1) {
            fn(0);
            return;
        }
        if (getpid() != pid_) {  // after a fork the parent's workers do not exist here, and its mutex and condition
            s_ = new State();    // variables remember waiters that are not there: start afresh, leave the old state alone
            pid_ = getpid();
        }
        State* s = s_;
        {
            std::lock_guard<std::mutex> hold(s->m);
            while (s->workers.size() < nt - 1) {
                const uint32_t id = (uint32_t)s->workers.size() + 1;
                const uint64_t before = s->gen;  // a worker that starts late still sees this run as new
                s->workers.emplace_back([s, id, before] { work(s, id, before); });
            }
            s->fn = &fn;
            s->active = nt;
            s->pending = nt - 1;
            s->gen++;
        }
        s->start.notify_all();
        fn(0);
        std::unique_lock<std::mutex> hold(s->m);
        s->done.wait(hold, [s] { return s->pending == 0; });
        s->fn = nullptr;
    }

  private:
    struct State {
        std::mutex m;
        std::condition_variable start, done;
        std::vector<std::thread> workers;
        const std::function<void(uint32_t)>* fn = nullptr;
        uint64_t gen = 0;
        uint32_t active = 0, pending = 0;
        bool stop = false;
    };
    static void work(State* s, uint32_t id, uint64_t seen) {
        for (;;) {
            const std::function<void(uint32_t)>* fn = nullptr;
            {
                std::unique_lock<std::mutex> hold(s->m);
                s->start.wait(hold, [&] { return s->gen != seen; });
                seen = s->gen;
                if (s->stop) return;
                if (id < s->active) fn = s->fn;
            }
            if (fn) {
                (*fn)(id);
                std::lock_guard<std::mutex> hold(s->m);
                if (--s->pending == 0) s->done.notify_one();
            }
        }
    }
    State* s_ = new State();
    pid_t pid_ = getpid();
};
static HostPool& host_pool() {
    static thread_local HostPool pool;
    return pool;
}

// One 64-vector word of a mask row: bit j set iff the 8 mask bytes of vector v0 + j hold a non-zero byte.
// `vn` ≤ 64 vectors exist from v0 on.
static inline uint64_t live_word_scalar(const uint8_t* m, uint32_t vn) {
    uint64_t bits = 0;
    for (uint32_t j = 0; j < vn; j++) {
        uint64_t m8;
        memcpy(&m8, m + (uint64_t)j * kVec, 8);
        bits |= (uint64_t)(m8 != 0) << j;
    }
    return bits;
}
// The same for a full word (512 mask bytes) with 32-byte compares, on CPUs that have AVX2 (looked up once).
__attribute__((target("avx2"))) static inline uint64_t live_word_avx2(const uint8_t* m) {
    const __m256i zero = _mm256_setzero_si256();
    uint64_t zeros = 0;
    for (int k = 0; k < 16; k++) {
        const __m256i v = _mm256_loadu_si256((const __m256i*)(m + 32 * k));
        zeros |= (uint64_t)(uint32_t)_mm256_movemask_pd(_mm256_castsi256_pd(_mm256_cmpeq_epi64(v, zero))) << (4 * k);
    }
    return ~zeros;
}
static bool host_has_avx2() {
    static const bool yes = __builtin_cpu_supports("avx2");
    return yes;
}

// Rows [r0, r1) of a chunk. First pass (`gather` false): the liveness words and the count of live vectors per row.
// Second pass: the live vectors' logits, reference logits and mask bytes to their places in the packed arrays; the
// row's live vectors are listed first, so that the lines of the vectors a few places ahead can be requested while
// the current ones are copied (the reads are scattered over 2 × 256 KB per row: without the requests a thread waits
// for one cache miss after another).
template <int ESIZE, bool REF>
static void pack_rows_range(const nrl_pack_args* a, uint64_t r0, uint64_t r1, uint32_t words_per_row, bool gather) {
    const uint32_t nvec = a->V / kVec;
    const bool avx2 = host_has_avx2();
    std::vector<uint16_t> list;  // V ≤ 262 144: vector indices fit 16 bits
    constexpr uint32_t kAheadVectors = 24;
    if (gather) list.resize((size_t)nvec + kAheadVectors);
    for (uint64_t r = r0; r < r1; r++) {
        const uint8_t* mrow = a->allow_mask + r * a->V;
        uint64_t* words = a->live_words + r * words_per_row;
        if (!gather) {
            uint32_t live = 0;
            for (uint32_t w = 0; w < words_per_row; w++) {
                const uint32_t v0 = w * 64, vn = nvec - v0 < 64u ? nvec - v0 : 64u;
                const uint64_t bits = (avx2 && vn == 64u) ? live_word_avx2(mrow + (uint64_t)v0 * kVec) : live_word_scalar(mrow + (uint64_t)v0 * kVec, vn);
                words[w] = bits;
                live += (uint32_t)__builtin_popcountll(bits);
            }
            a->row_offset[r + 1] = live;  // counts for now; the caller turns them into offsets
        } else {
            uint32_t n = 0;
            for (uint32_t w = 0; w < words_per_row; w++) {
                uint64_t bits = words[w];
                while (bits) {
                    list[n++] = (uint16_t)(w * 64 + (uint32_t)__builtin_ctzll(bits));
                    bits &= bits - 1;
                }
            }
            for (uint32_t k = 0; k < kAheadVectors; k++) list[n + k] = n ? list[n - 1] : 0;  // requests past the end go to a line already held
            const char* xrow = (const char*)a->logits + r * a->V * ESIZE;
            const char* rrow = REF ? (const char*)a->ref_logits + r * a->V * ESIZE : nullptr;
            char* px = (char*)a->packed_logits + (uint64_t)a->row_offset[r] * (kVec * ESIZE);
            char* pr = REF ? (char*)a->packed_ref + (uint64_t)a->row_offset[r] * (kVec * ESIZE) : nullptr;
            uint64_t* pm = a->packed_mask + a->row_offset[r];
            for (uint32_t k = 0; k < n; k++) {
                const uint64_t ahead = list[k + kAheadVectors], v = list[k];
                _mm_prefetch(xrow + ahead * (kVec * ESIZE), _MM_HINT_T0);
                if (REF) _mm_prefetch(rrow + ahead * (kVec * ESIZE), _MM_HINT_T0);
                _mm_prefetch((const char*)mrow + ahead * kVec, _MM_HINT_T0);
                if (ESIZE == 4) {
                    _mm_prefetch(xrow + ahead * (kVec * ESIZE) + 16, _MM_HINT_T0);  // a 32-byte vector can straddle two lines
                    if (REF) _mm_prefetch(rrow + ahead * (kVec * ESIZE) + 16, _MM_HINT_T0);
                }
                for (int q = 0; q < kVec * ESIZE / 16; q++) {
                    _mm_storeu_si128((__m128i*)(px + (uint64_t)k * (kVec * ESIZE)) + q, _mm_loadu_si128((const __m128i*)(xrow + v * (kVec * ESIZE)) + q));
                    if (REF) _mm_storeu_si128((__m128i*)(pr + (uint64_t)k * (kVec * ESIZE)) + q, _mm_loadu_si128((const __m128i*)(rrow + v * (kVec * ESIZE)) + q));
                }
                memcpy(pm + k, mrow + v * kVec, 8);
            }
        }
    }
}

template <int ESIZE, bool REF>
static int host_pack_impl(nrl_pack_args* a) {
    const uint32_t nvec = a->V / kVec, words_per_row = (nvec + 63) / 64;
    const uint32_t nt = a->threads < 1 ? 1 : (a->threads > 256 ? 256 : a->threads);
    const uint64_t per = (a->rows + nt - 1) / nt;
    auto run = [&](bool gather) {
        host_pool().run(nt, [&](uint32_t t) {
            const uint64_t r0 = t * per < a->rows ? t * per : a->rows, r1 = (t + 1) * per < a->rows ? (t + 1) * per : a->rows;
            if (r0 < r1) pack_rows_range<ESIZE, REF>(a, r0, r1, words_per_row, gather);
        });
    };
    run(false);
    a->row_offset[0] = 0;
    uint64_t total = 0;
    for (uint64_t r = 0; r < a->rows; r++) {
        total += a->row_offset[r + 1];
        if (total > 0xffffffffull) return NRL_E_UNSUPPORTED;
        a->row_offset[r + 1] = (uint32_t)total;
    }
    a->live_vectors = total;
    if (total > a->capacity) return NRL_E_WORKSPACE;
    run(true);
    return NRL_OK;
}

// A byte mask to a bit mask on the host (bit v of a row = bit v mod 32 of its word v / 32): 16
// mask bytes per SSE2 compare. What the bit-mask kernels (NRL_FWD_MASK_BITS) then read is an
// eighth of the bytes, which is what counts when the mask has to cross the host link.
static void pack_bits_range(const uint8_t* mask, uint32_t* bits, uint64_t r0, uint64_t r1, uint32_t V, uint32_t words) {
    const __m128i zero = _mm_setzero_si128();
    for (uint64_t r = r0; r < r1; r++) {
        const uint8_t* m = mask + r * V;
        uint32_t* out = bits + r * words;
        const uint32_t full = V / 32;
        for (uint32_t w = 0; w < full; w++) {
            const __m128i a = _mm_loadu_si128((const __m128i*)(m + 32 * w));
            const __m128i b = _mm_loadu_si128((const __m128i*)(m + 32 * w + 16));
            const uint32_t za = (uint32_t)_mm_movemask_epi8(_mm_cmpeq_epi8(a, zero));
            const uint32_t zb = (uint32_t)_mm_movemask_epi8(_mm_cmpeq_epi8(b, zero));
            out[w] = ~(za | (zb << 16));
        }
        if (full < words) {
            uint32_t x = 0;
            for (uint32_t v = full * 32; v < V; v++) x |= (uint32_t)(m[v] != 0) << (v & 31u);
            out[full] = x;
        }
    }
}

static int host_pack_bits_impl(uint64_t rows, uint32_t V, const uint8_t* mask, uint32_t* bits, uint32_t threads) {
    const uint32_t words = (V + 31) / 32;
    const uint32_t nt = threads < 1 ? 1 : (threads > 256 ? 256 : threads);
    const uint64_t per = (rows + nt - 1) / nt;
    host_pool().run(nt, [&](uint32_t t) {
        const uint64_t r0 = t * per < rows ? t * per : rows, r1 = (t + 1) * per < rows ? (t + 1) * per : rows;
        if (r0 < r1) pack_bits_range(mask, bits, r0, r1, V, words);
    });
    return NRL_OK;
}

// One block per row. Warp w takes the row's 64-vector words w, w + 8, …; lane l the vectors
// 2l and 2l + 1 of a word: their mask bytes are one 16-byte store, their logits two.
template <int ESIZE, bool REF>
__global__ void __launch_bounds__(256) unpack_rows_kernel(uint32_t V, const uint64_t* live_words, const uint32_t* row_offset, const uint4* packed_logits,
                                                          const uint4* packed_ref, const uint2* packed_mask, char* logits, char* ref, uint8_t* mask) {
    __shared__ uint32_t before[512 + 1];  // live vectors of the row before each word
    const uint64_t row = blockIdx.x;
    const uint32_t nvec = V / kVec, words = (nvec + 63) / 64;
    const uint64_t* wrow = live_words + row * words;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t w = threadIdx.x; w < words; w += blockDim.x) before[w + 1] = (uint32_t)__popcll(wrow[w]);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = row_offset[row];
        for (uint32_t w = 0; w < words; w++) {
            const uint32_t c = before[w + 1];
            before[w] = run;
            run += c;
        }
    }
    __syncthreads();
    constexpr uint32_t kPieces = kVec * ESIZE / 16;  // 16-byte pieces of one vector of logits
    for (uint32_t w = warp; w < words; w += blockDim.x / 32) {
        const uint64_t bits = wrow[w];
        const uint32_t v = w * 64 + 2 * lane;  // this lane's first vector
        if (v >= nvec) continue;
        const uint32_t pair = (uint32_t)(bits >> (2 * lane)) & 3u;
        uint32_t idx = before[w] + (uint32_t)__popcll(bits & ((1ull << (2 * lane)) - 1ull));
        uint2 m0 = make_uint2(0u, 0u), m1 = make_uint2(0u, 0u);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            if (!((pair >> h) & 1u) || v + h >= nvec) continue;
            const uint2 mk = packed_mask[idx];
            if (h == 0) m0 = mk; else m1 = mk;
            const uint64_t dst = (row * V + (uint64_t)(v + h) * kVec) * ESIZE;
#pragma unroll
            for (uint32_t k = 0; k < kPieces; k++) {
                *reinterpret_cast<uint4*>(logits + dst + 16 * k) = packed_logits[(uint64_t)idx * kPieces + k];
                if (REF) *reinterpret_cast<uint4*>(ref + dst + 16 * k) = packed_ref[(uint64_t)idx * kPieces + k];
            }
            idx++;
        }
        // a mask row starts on a 16-byte boundary only when V is a multiple of 16
        uint8_t* mdst = mask + row * V + (uint64_t)v * kVec;
        if (v + 1 < nvec && (reinterpret_cast<uintptr_t>(mdst) & 15u) == 0) {
            *reinterpret_cast<uint4*>(mdst) = make_uint4(m0.x, m0.y, m1.x, m1.y);
        } else {
            *reinterpret_cast<uint2*>(mdst) = m0;
            if (v + 1 < nvec) *reinterpret_cast<uint2*>(mdst + 8) = m1;
        }
    }
}

// Bit-packed vocabulary masks: bit v of a row is bit (v mod 32) of its 32-bit word v / 32 (the
// layout grammar engines emit). One thread expands one byte of bits into eight mask bytes.
__global__ void __launch_bounds__(256) expand_bitmask_kernel(uint64_t rows, uint32_t V, uint32_t words_per_row, uint64_t bits_row_stride_words, const uint32_t* __restrict__ bits,
                                                             uint8_t* __restrict__ out) {
    const uint32_t bytes_per_row = (V + 7) / 8;
    const uint64_t total = rows * bytes_per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / bytes_per_row;
        const uint32_t b = (uint32_t)(i - row * bytes_per_row);  // byte of bits within the row
        const uint32_t w = __ldg(bits + row * bits_row_stride_words + (b >> 2));
        const uint32_t byte = (w >> (8 * (b & 3))) & 0xffu;
        // spread bit k of `byte` to byte k: 0 or 1
        const uint32_t lo = ((byte & 0xfu) * 0x00204081u) & 0x01010101u;
        const uint32_t hi = ((byte >> 4) * 0x00204081u) & 0x01010101u;
        uint8_t* dst = out + row * V + (uint64_t)b * 8;
        const uint32_t left = V - b * 8;
        if (left >= 8 && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
        } else {
            for (uint32_t k = 0; k < 8 && k < left; k++) dst[k] = (uint8_t)((byte >> k) & 1u);
        }
    }
    (void)words_per_row;
}

}  // namespace nrl
