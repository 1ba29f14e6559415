// Token-level losses over [S, B, T] values and the TokenReduction kernels. These touch rows,
// not rows·V, elements: their cost is launch latency. Every sum runs in a fixed order.
#pragma once
#include "common.cuh"

namespace nrl {

struct TokParams {
    const float* logp;
    const float* other;
    const float* weights;
    const float* mask;
    const float* upstream;
    float* loss;
    float* dloss;
    uint64_t n;  // S·B·T
    uint64_t T;
    uint32_t kind;
    uint32_t w_per_seq;
    uint32_t has_dual;
    uint32_t has_clamp;
    uint32_t accumulate;  // dloss += instead of =
    float ratio_lo, ratio_hi;  // (f32)(1 − low), (f32)(1 + high)
    float neg_dual;            // (f32)(−c)
    float clamp;
};

// clamp(x, −b, b) as the reference builds it: clamp_max then clamp_min, each a mask_fill of a
// comparison (src/tensor/float.rs:578-594); `pass` is false where a bound replaced the value.
__device__ __forceinline__ float clamp_sym(float x, float b, bool& pass) {
    pass = true;
    if (x > b) { x = b; pass = false; }
    if (x < -b) { x = -b; pass = false; }
    return x;
}

// One position of a token-level loss: the value `per` and d per / d logp `dl` (both exactly 0 at
// an unscored position: zero_masked is a select, so garbage there never leaks).
__device__ __forceinline__ void token_loss_eval(const TokParams& p, uint64_t i, bool scored, float& per, float& dl) {
    const float lp = p.logp[i];
    per = 0.f;
    dl = 0.f;
    if (p.kind == NRL_LOSS_PG) {
        float w = p.weights[p.w_per_seq ? i / p.T : i];
        per = -(lp * w);
        dl = -w;
    } else if (p.kind == NRL_LOSS_PPO) {
        float a = p.weights[p.w_per_seq ? i / p.T : i];
        float d = scored ? lp - p.other[i] : 0.f;  // log_ratio zeroes unscored positions first
        bool pass_d = true;
        if (p.has_clamp) d = clamp_sym(d, p.clamp, pass_d);
        float r = expf(d);
        float unclipped = -(r * a);
        float rc = r;
        bool pass_r = true;
        if (rc > p.ratio_hi) { rc = p.ratio_hi; pass_r = false; }
        if (rc < p.ratio_lo) { rc = p.ratio_lo; pass_r = false; }
        float clipped = -(rc * a);
        bool u_wins = (unclipped - clipped) > 0.f;  // select_max: a tie or NaN takes the clipped branch
        float ppo = u_wins ? unclipped : clipped;
        float g_ppo = 1.f;  // upstream of ppo
        per = ppo;
        if (p.has_dual) {
            float cap = a * p.neg_dual;                 // −c·A
            bool ppo_side = ((-ppo) - (-cap)) > 0.f;    // select_max(−ppo, −cap)
            float capped = -(ppo_side ? -ppo : -cap);   // min(ppo, −c·A)
            if (a < 0.f) {
                per = capped;
                g_ppo = ppo_side ? 1.f : 0.f;
            }
        }
        // d per / d r through the two branches of select_max, then exp's g·y
        float g_u = u_wins ? g_ppo : 0.f, g_c = u_wins ? 0.f : g_ppo;
        float g_r = (-g_u) * a + (pass_r ? (-g_c) * a : 0.f);
        float g_d = g_r * r;
        dl = pass_d ? g_d : 0.f;
    } else {
        float d = scored ? p.other[i] - lp : 0.f;  // δ = ref − logp
        bool pass_d = true;
        if (p.has_clamp) d = clamp_sym(d, p.clamp, pass_d);
        float g_d;
        if (p.kind == NRL_LOSS_K1) {
            per = -d;
            g_d = -1.f;
        } else if (p.kind == NRL_LOSS_K2) {
            per = (d * d) / 2.0f;
            g_d = d;
        } else {
            float e = expf(d);
            per = e - (d + 1.0f);
            g_d = e + (-1.f);
        }
        dl = pass_d ? -g_d : 0.f;
    }
    if (!scored) { per = 0.f; dl = 0.f; }
}

__global__ void token_loss_kernel(TokParams p) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    const bool scored = p.mask ? (p.mask[i] != 0.f) : true;
    float per, dl;
    token_loss_eval(p, i, scored, per, dl);
    if (p.loss) p.loss[i] = per;
    if (p.dloss) {
        float d = (p.upstream && scored) ? p.upstream[i] * dl : dl;
        p.dloss[i] = p.accumulate ? p.dloss[i] + d : d;
    }
}

// block-wide sum of (a, b) in a fixed tree; result valid on thread 0
template <int NT>
__device__ __forceinline__ void block_sum2(float& a, float& b, float* sm) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, s);
        b += __shfl_xor_sync(0xffffffffu, b, s);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { sm[warp] = a; sm[NT / 32 + warp] = b; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float x = 0.f, y = 0.f;
        for (int w = 0; w < NT / 32; w++) { x += sm[w]; y += sm[NT / 32 + w]; }
        a = x; b = y;
    }
}

constexpr int kRedThreads = 256;

// clip_fraction (src/nn/rl.rs:293-317): one block per seed.
__global__ void __launch_bounds__(kRedThreads) clip_fraction_kernel(TokParams p, uint64_t per_seed, float* out) {
    __shared__ float sm[2 * kRedThreads / 32];
    const uint64_t s = blockIdx.x;
    float hits = 0.f, cnt = 0.f;
    for (uint64_t j = threadIdx.x; j < per_seed; j += kRedThreads) {
        uint64_t i = s * per_seed + j;
        float mk = p.mask ? p.mask[i] : 1.f;
        bool scored = mk != 0.f;
        float a = p.weights[p.w_per_seq ? i / p.T : i];
        float d = scored ? p.logp[i] - p.other[i] : 0.f;
        float r = expf(d);
        float pos = a > 0.f ? 1.f : 0.f, neg = a < 0.f ? 1.f : 0.f;
        float hit = (r > p.ratio_hi ? 1.f : 0.f) * pos + (r < p.ratio_lo ? 1.f : 0.f) * neg;
        if (p.has_dual) hit = hit + (r > -p.neg_dual ? 1.f : 0.f) * neg;
        if (p.has_clamp) hit = hit + (fabsf(d) > p.clamp ? 1.f : 0.f);
        if (hit > 1.f) hit = 1.f;
        hits += hit * mk;
        cnt += mk;
    }
    block_sum2<kRedThreads>(hits, cnt, sm);
    if (threadIdx.x == 0) out[s] = hits / fmaxf(cnt, 1.f);
}

// ---- TokenReduction (src/nn/rl.rs:36-92) -----------------------------------------------------------
//
// Two fixed steps, the same whoever runs them: (1) one WARP sums a sequence — lane l adds the
// elements l, l + 32, … of the sequence in that order, then the 32 lane sums meet in a butterfly —
// giving the pair (Σ per, Σ mask) of that sequence; (2) a seed's pairs are folded in sequence order
// in f64. nrl_reduce_tokens does both in one kernel (a block per seed, its warps taking the
// seed's sequences side by side); callers whose sequences are spread over several GPUs run step
// 1 where the sequences live (seq_pairs_kernel), gather the pairs and run step 2
// (fold_pairs_kernel): the bits are the same for any number of GPUs.
constexpr int kFoldThreads = 1024;  // 32 warps per seed
constexpr int kSeqChunk = 1024;     // sequences of a seed held in shared memory between the two steps

__device__ __forceinline__ void seq_sum(const float* __restrict__ per, const float* __restrict__ mask, uint64_t base, uint64_t T, float& v, float& c) {
    const int lane = threadIdx.x & 31;
    v = 0.f;
    c = 0.f;
    for (uint64_t t = lane; t < T; t += 32) {
        if (per) v += per[base + t];
        c += mask ? mask[base + t] : 1.f;
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, s);
        c += __shfl_xor_sync(0xffffffffu, c, s);
    }
}

struct SeedFold {
    double tot = 0.0, count = 0.0, seq_tot = 0.0, nonempty = 0.0;
    __device__ __forceinline__ void add(float v, float c) {
        tot += (double)v;
        count += (double)c;
        seq_tot += (double)(v / fmaxf(c, 1.f));  // per_sequence (src/nn/rl.rs:88-92)
        nonempty += (double)fminf(c, 1.f);
    }
    __device__ __forceinline__ float value(uint32_t reduction) const {
        if (reduction == NRL_REDUCE_SUM) return (float)tot;
        if (reduction == NRL_REDUCE_TOKEN_MEAN) return (float)tot / fmaxf((float)count, 1.f);
        return (float)seq_tot / fmaxf((float)nonempty, 1.f);  // SEQUENCE_MEAN
    }
    __device__ __forceinline__ float scale(uint32_t reduction) const {
        if (reduction == NRL_REDUCE_TOKEN_MEAN) return fmaxf((float)count, 1.f);
        if (reduction == NRL_REDUCE_SEQUENCE_MEAN) return fmaxf((float)nonempty, 1.f);
        return 1.f;
    }
};

// One block per seed: both steps.
__global__ void __launch_bounds__(kFoldThreads) reduce_tokens_kernel(uint32_t reduction, uint64_t B, uint64_t T, const float* per, const float* mask, float* out) {
    __shared__ float sv[kSeqChunk], sc[kSeqChunk];
    const uint64_t s = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    SeedFold f;
    for (uint64_t b0 = 0; b0 < B; b0 += kSeqChunk) {
        const int n = (int)(B - b0 < (uint64_t)kSeqChunk ? B - b0 : (uint64_t)kSeqChunk);
        for (int j = warp; j < n; j += kFoldThreads / 32) {
            float v, c;
            seq_sum(per, mask, (s * B + b0 + j) * T, T, v, c);
            if (lane == 0) {
                sv[j] = v;
                sc[j] = c;
                if (reduction == NRL_REDUCE_PER_SEQUENCE) out[s * B + b0 + j] = v / fmaxf(c, 1.f);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0 && reduction != NRL_REDUCE_PER_SEQUENCE)
            for (int j = 0; j < n; j++) f.add(sv[j], sc[j]);
        __syncthreads();
    }
    if (threadIdx.x == 0 && reduction != NRL_REDUCE_PER_SEQUENCE) out[s] = f.value(reduction);
}

// Step 1 alone: pairs[q] = (Σ per, Σ mask) of sequence q, one warp each.
__global__ void __launch_bounds__(256) seq_pairs_kernel(uint64_t n_seq, uint64_t T, const float* per, const float* mask, float2* pairs) {
    const uint64_t q = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (q >= n_seq) return;
    float v, c;
    seq_sum(per, mask, q * T, T, v, c);
    if ((threadIdx.x & 31) == 0) pairs[q] = make_float2(v, c);
}

// Step 2 alone: one thread per seed folds its B pairs in sequence order (PER_SEQUENCE: one thread per sequence).
__global__ void fold_pairs_kernel(uint32_t reduction, uint64_t S, uint64_t B, const float2* pairs, float* out) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (reduction == NRL_REDUCE_PER_SEQUENCE) {
        if (i < S * B) out[i] = pairs[i].x / fmaxf(pairs[i].y, 1.f);
        return;
    }
    if (i >= S) return;
    SeedFold f;
    for (uint64_t b = 0; b < B; b++) f.add(pairs[i * B + b].x, pairs[i * B + b].y);
    out[i] = f.value(reduction);
}

// TokenReduction backward: d_per from the reduced value's upstream gradient. One block per seed:
// the seed's divisor first (the counts of all its sequences, folded as in the forward), then its
// warps write the sequences side by side.
__global__ void __launch_bounds__(kFoldThreads) reduce_tokens_bwd_kernel(uint32_t reduction, uint64_t B, uint64_t T, const float* mask, const float* g_out, float* d_per) {
    __shared__ float sc[kSeqChunk];
    __shared__ float sh_scale;
    const uint64_t s = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float seed_scale = 1.f;
    if (reduction == NRL_REDUCE_TOKEN_MEAN || reduction == NRL_REDUCE_SEQUENCE_MEAN) {
        SeedFold f;
        for (uint64_t b0 = 0; b0 < B; b0 += kSeqChunk) {
            const int n = (int)(B - b0 < (uint64_t)kSeqChunk ? B - b0 : (uint64_t)kSeqChunk);
            for (int j = warp; j < n; j += kFoldThreads / 32) {
                float v, c;
                seq_sum(nullptr, mask, (s * B + b0 + j) * T, T, v, c);
                if (lane == 0) sc[j] = c;
            }
            __syncthreads();
            if (threadIdx.x == 0)
                for (int j = 0; j < n; j++) f.add(0.f, sc[j]);
            __syncthreads();
        }
        if (threadIdx.x == 0) sh_scale = f.scale(reduction);
        __syncthreads();
        seed_scale = sh_scale;
    }
    for (uint64_t b = warp; b < B; b += kFoldThreads / 32) {
        const uint64_t base = (s * B + b) * T;
        float g = 0.f;
        if (reduction == NRL_REDUCE_PER_SEQUENCE || reduction == NRL_REDUCE_SEQUENCE_MEAN) {
            float v, c;
            seq_sum(nullptr, mask, base, T, v, c);
            const float seq_scale = fmaxf(c, 1.f);
            g = reduction == NRL_REDUCE_PER_SEQUENCE ? g_out[s * B + b] / seq_scale : (g_out[s] / seed_scale) / seq_scale;
        } else if (reduction == NRL_REDUCE_TOKEN_MEAN) {
            g = g_out[s] / seed_scale;
        } else if (reduction == NRL_REDUCE_SUM) {
            g = g_out[s];
        }
        for (uint64_t t = lane; t < T; t += 32) {
            const bool scored = mask ? mask[base + t] != 0.f : true;
            const float gi = reduction == NRL_REDUCE_NONE ? g_out[base + t] : g;
            d_per[base + t] = scored ? gi : 0.f;
        }
    }
}

// The same backward for a caller that holds only the sequences [seq_begin, seq_begin + n_seq) of
// the job: the counts come from the gathered pairs of ALL sequences, `mask` and `d_per` cover
// the local sequences, `g_out` is the whole reduced value's gradient ([S] or [S, B]; for NONE the
// local [n_seq, T]). One warp per local sequence.
__global__ void __launch_bounds__(256) reduce_tokens_bwd_pairs_kernel(uint32_t reduction, uint64_t B, uint64_t T, uint64_t seq_begin, uint64_t n_seq,
                                                                      const float2* pairs, const float* mask, const float* g_out, float* d_per) {
    const uint64_t q = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (q >= n_seq) return;
    const int lane = threadIdx.x & 31;
    const uint64_t seq = seq_begin + q, s = seq / B;
    float g = 0.f;
    if (reduction != NRL_REDUCE_NONE) {
        float seed_scale = 1.f;
        if (reduction == NRL_REDUCE_TOKEN_MEAN || reduction == NRL_REDUCE_SEQUENCE_MEAN) {
            SeedFold f;
            for (uint64_t b = 0; b < B; b++) f.add(0.f, pairs[s * B + b].y);
            seed_scale = f.scale(reduction);
        }
        const float seq_scale = fmaxf(pairs[seq].y, 1.f);
        if (reduction == NRL_REDUCE_PER_SEQUENCE) g = g_out[seq] / seq_scale;
        else if (reduction == NRL_REDUCE_SEQUENCE_MEAN) g = (g_out[s] / seed_scale) / seq_scale;
        else if (reduction == NRL_REDUCE_TOKEN_MEAN) g = g_out[s] / seed_scale;
        else g = g_out[s];
    }
    const uint64_t base = q * T;
    for (uint64_t t = lane; t < T; t += 32) {
        const bool scored = mask ? mask[base + t] != 0.f : true;
        const float gi = reduction == NRL_REDUCE_NONE ? g_out[base + t] : g;
        d_per[base + t] = scored ? gi : 0.f;
    }
}

// ---- a whole token-level objective in one launch ---------------------------------------------------
//
// A PPO-style step reduces three per-token quantities with the same TokenReduction — the clipped
// policy loss of the log-probs, the exact KL and the entropy the row forward left per token — and
// then needs, per token, the upstream gradients the row backward takes. Done with the separate
// entry points that is one token_loss, three reduce_tokens, three reduce_tokens_bwd and one more
// token_loss launch. This kernel does all of it per seed (one block, warps taking the seed's
// sequences side by side): step 1 sums each sequence of the three quantities and folds the
// sequences in order — the very operations of reduce_tokens_kernel, so the reduced values have
// its bits; step 2 writes g_logp = d_per · d loss / d logp, g_kl = d_per_kl and g_ent = d_per_ent,
// with d_per the values reduce_tokens_bwd_kernel would write (same divisions).
struct ObjectiveParams {
    TokParams tok;            // the policy term (logp, other, weights, mask, clip constants); n = S·B·T
    const float* kl;          // per-token exact KL [S,B,T] or null
    const float* entropy;     // per-token entropy [S,B,T] or null
    const float* up_policy;   // upstream gradients of the three reduced values, [S] each; null = ones
    const float* up_kl;
    const float* up_entropy;
    float* out_policy;        // reduced values [S]
    float* out_kl;
    float* out_entropy;
    float* g_logp;            // per-token gradients for nrl_row_bwd, [S,B,T]
    float* g_kl;
    float* g_ent;
    uint64_t B, T;
    uint32_t reduction;       // SUM, TOKEN_MEAN or SEQUENCE_MEAN
};

__global__ void __launch_bounds__(kFoldThreads) token_objective_kernel(ObjectiveParams p) {
    __shared__ float sv[3][kSeqChunk], sc[kSeqChunk];
    __shared__ float sh_scale;
    const uint64_t s = blockIdx.x, B = p.B, T = p.T;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* mask = p.tok.mask;
    SeedFold f[3];
    for (uint64_t b0 = 0; b0 < B; b0 += kSeqChunk) {
        const int n = (int)(B - b0 < (uint64_t)kSeqChunk ? B - b0 : (uint64_t)kSeqChunk);
        for (int j = warp; j < n; j += kFoldThreads / 32) {
            const uint64_t base = (s * B + b0 + j) * T;
            // seq_sum's order: lane l adds its elements l, l + 32, … then the butterfly
            float v0 = 0.f, v1 = 0.f, v2 = 0.f, c = 0.f;
            for (uint64_t t = lane; t < T; t += 32) {
                const uint64_t i = base + t;
                const bool scored = mask ? mask[i] != 0.f : true;
                float per, dl;
                token_loss_eval(p.tok, i, scored, per, dl);
                v0 = __fadd_rn(v0, per);  // never contracted with the loss's last product: the sum of the stored values
                if (p.kl) v1 += scored ? p.kl[i] : 0.f;          // zero_masked, then the reduction
                if (p.entropy) v2 += scored ? p.entropy[i] : 0.f;
                c += mask ? mask[i] : 1.f;
            }
#pragma unroll
            for (int k = 16; k >= 1; k >>= 1) {
                v0 += __shfl_xor_sync(0xffffffffu, v0, k);
                v1 += __shfl_xor_sync(0xffffffffu, v1, k);
                v2 += __shfl_xor_sync(0xffffffffu, v2, k);
                c += __shfl_xor_sync(0xffffffffu, c, k);
            }
            if (lane == 0) { sv[0][j] = v0; sv[1][j] = v1; sv[2][j] = v2; sc[j] = c; }
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int j = 0; j < n; j++) { f[0].add(sv[0][j], sc[j]); f[1].add(sv[1][j], sc[j]); f[2].add(sv[2][j], sc[j]); }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (p.out_policy) p.out_policy[s] = f[0].value(p.reduction);
        if (p.kl && p.out_kl) p.out_kl[s] = f[1].value(p.reduction);
        if (p.entropy && p.out_entropy) p.out_entropy[s] = f[2].value(p.reduction);
        sh_scale = f[0].scale(p.reduction);
    }
    __syncthreads();
    if (!p.g_logp && !p.g_kl && !p.g_ent) return;
    const float seed_scale = sh_scale;
    const float up0 = p.up_policy ? p.up_policy[s] : 1.f, up1 = p.up_kl ? p.up_kl[s] : 1.f, up2 = p.up_entropy ? p.up_entropy[s] : 1.f;
    for (uint64_t b = warp; b < B; b += kFoldThreads / 32) {
        const uint64_t base = (s * B + b) * T;
        float seq_scale = 1.f;
        if (p.reduction == NRL_REDUCE_SEQUENCE_MEAN) {
            float v, c;
            seq_sum(nullptr, mask, base, T, v, c);
            seq_scale = fmaxf(c, 1.f);
        }
        // d_per of reduce_tokens_bwd_kernel for each of the three upstreams
        float d0, d1, d2;
        if (p.reduction == NRL_REDUCE_SEQUENCE_MEAN) { d0 = (up0 / seed_scale) / seq_scale; d1 = (up1 / seed_scale) / seq_scale; d2 = (up2 / seed_scale) / seq_scale; }
        else if (p.reduction == NRL_REDUCE_TOKEN_MEAN) { d0 = up0 / seed_scale; d1 = up1 / seed_scale; d2 = up2 / seed_scale; }
        else { d0 = up0; d1 = up1; d2 = up2; }
        for (uint64_t t = lane; t < T; t += 32) {
            const uint64_t i = base + t;
            const bool scored = mask ? mask[i] != 0.f : true;
            if (p.g_logp) {
                float per, dl;
                token_loss_eval(p.tok, i, scored, per, dl);
                p.g_logp[i] = scored ? d0 * dl : dl;  // token_loss_kernel's `upstream · dl` (dl is 0 where unscored)
            }
            if (p.g_kl) p.g_kl[i] = scored ? d1 : 0.f;
            if (p.g_ent) p.g_ent[i] = scored ? d2 : 0.f;
        }
    }
}

// check_scored_finite (src/nn/rl.rs:204-211) on the device: the first flat position whose mask is
// non-zero (no mask: every position) and whose value is not finite. One block; a thread keeps
// the smallest such index of its strided share, the block takes the minimum in a fixed tree (a
// minimum does not depend on the order anyway). out[0] = the index or ~0, out[1] = the value's bits.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads) first_nonfinite_kernel(uint64_t n, const float* x, const float* mask, uint64_t* out) {
    __shared__ uint64_t sm[kScanThreads / 32];
    uint64_t first = ~0ull;
    for (uint64_t i = threadIdx.x; i < n && first == ~0ull; i += kScanThreads) {
        const float v = x[i];
        const bool scored = mask ? mask[i] != 0.f : true;
        if (scored && !(fabsf(v) <= FLT_MAX)) first = i;
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const uint64_t o = __shfl_xor_sync(0xffffffffu, first, s);
        first = o < first ? o : first;
    }
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = first;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kScanThreads / 32; w++) first = sm[w] < first ? sm[w] : first;
        out[0] = first;
        out[1] = first == ~0ull ? 0ull : (uint64_t)__float_as_uint(x[first]);
    }
}

__global__ void mask_rows_kernel(uint64_t n, const float* x, const float* mask, float* out) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (mask && mask[i] == 0.f) ? 0.f : x[i];
}

// group_advantages (src/nn/rl.rs:436-461) on the device, in the host's own f64 operand order so
// that the result is the reference's bit for bit: per group of n rewards min/max (all equal →
// exact zeros), the left-to-right sum, mean, optionally the left-to-right sum of squared
// deviations → standard deviation + eps, then (r − mean) / scale, rounded to f32 once. One thread
// per group; products and sums are written with explicit roundings so nothing is fused.
__global__ void group_advantages_kernel(uint64_t groups, uint32_t n, int norm_std, double eps, int unbiased, const float* rewards, float* out) {
    const uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const float* r = rewards + g * n;
    float* o = out + g * n;
    double lo = (double)__int_as_float(0x7f800000), hi = -lo, sum = 0.0;
    for (uint32_t i = 0; i < n; i++) {
        const double x = (double)r[i];
        lo = fmin(lo, x);
        hi = fmax(hi, x);
        sum = __dadd_rn(sum, x);
    }
    if (lo == hi) {
        for (uint32_t i = 0; i < n; i++) o[i] = 0.f;
        return;
    }
    const double mean = __ddiv_rn(sum, (double)n);
    double scale = 1.0;
    if (norm_std) {
        double ss = 0.0;
        for (uint32_t i = 0; i < n; i++) {
            const double d = __dsub_rn((double)r[i], mean);
            ss = __dadd_rn(ss, __dmul_rn(d, d));
        }
        const double var = __ddiv_rn(ss, unbiased ? (double)(n - 1) : (double)n);
        scale = __dadd_rn(__dsqrt_rn(var), eps);
    }
    for (uint32_t i = 0; i < n; i++) o[i] = (float)__ddiv_rn(__dsub_rn((double)r[i], mean), scale);
}

}  // namespace nrl
