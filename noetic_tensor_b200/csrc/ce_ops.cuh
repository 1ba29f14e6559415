// The O(rows) and row-sum parts of the cross-entropy family over the row kernels: the per-row
// sum of the logits (label smoothing needs −mean_v log π_v = m + ln Z − Σ_v z_v / V) and the
// per-position loss with its two per-row upstream gradients.
#pragma once
#include "common.cuh"

namespace nrl {

constexpr int kSumThreads = 256;

// out[row] = Σ_v logits[row, v] in f32. One block per row; a thread adds its vectors in index
// order into 8 accumulators (one per position in the vector), which are added pairwise, then the
// block's 256 values in a fixed tree: the same result run to run.
template <int DT>
__global__ void __launch_bounds__(kSumThreads) row_sum_kernel(const void* logits, uint32_t V, bool vec, float* out) {
    __shared__ float sm[kSumThreads / 32];
    const uint64_t row = blockIdx.x;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    for (uint32_t v = threadIdx.x * kVec; v < V; v += kSumThreads * kVec) {
        Raw<DT> raw;
        float z[8];
        const int n = (int)min(V - v, (uint32_t)kVec);
        if (vec) raw.load(logits, row * V + v);
        else raw.load_scalar(logits, row * V + v, n);
        raw.unpack(z);
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (vec || i < n) acc[i] += z[i];
    }
    float s = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
#pragma unroll
    for (int k = 16; k >= 1; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kSumThreads / 32; w++) t += sm[w];
        out[row] = t;
    }
}

struct CeParams {
    const float* logp;
    const float* rowstats;
    const float* logit_sum;
    const float* keep;
    const float* upstream;
    float* loss;
    float* g_logp;
    float* g_uniform;
    uint64_t n;
    float eps, one_minus_eps, inv_v;
};

// loss = ((1 − ε)·nll + ε·uniform)·keep, a product as in the reference (src/nn/loss.rs:33, 78).
__global__ void ce_tokens_kernel(CeParams p) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    const float k = p.keep ? p.keep[i] : 1.f;
    if (p.loss) {
        float l = -p.logp[i];
        if (p.eps > 0.f) {
            const float4 st = reinterpret_cast<const float4*>(p.rowstats)[i];
            const float uniform = (st.x + st.y) - p.logit_sum[i] * p.inv_v;  // −mean_v log π_v
            l = l * p.one_minus_eps + uniform * p.eps;
        }
        p.loss[i] = l * k;
    }
    if (p.upstream) {
        const float g = p.upstream[i] * k;
        p.g_logp[i] = -(p.eps > 0.f ? p.one_minus_eps * g : g);
        if (p.g_uniform) p.g_uniform[i] = p.eps * g;
    }
}

}  // namespace nrl
