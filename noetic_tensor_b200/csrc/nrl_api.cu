// The C ABI of include/nrl.h: argument checking, kernel selection and launches. No allocation,
// no synchronisation (except nrl_check_status, which is a host read by definition).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "row_bwd.cuh"
#include "row_fwd_group.cuh"
#include "token_ops.cuh"
#include "ce_ops.cuh"
#include "gumbel.cuh"
#include "host_pack.cuh"
#include "lane_ops.cuh"
#include "readout.cuh"

#define NRL_STR2(x) #x
#define NRL_STR(x) NRL_STR2(x)
#ifndef NRL_SRC_HASH
#define NRL_SRC_HASH "unknown"
#endif

using namespace nrl;

std::atomic<uint64_t> nrl_g_launches{0};  // shared with the bit-mask translation unit
#define g_launches nrl_g_launches

static inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? NRL_OK : (int)e; }
static inline int after_launch(int n = 1) {
    g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed);
    return cuda_rc(cudaGetLastError());
}

extern "C" int nrl_version(void) { return 100; }

extern "C" const char* nrl_key(void) {
    // what results depend on: the target, the arithmetic options, the kernel sources
    return "cuda-sm100a-nvcc" NRL_STR(__CUDACC_VER_MAJOR__) "." NRL_STR(__CUDACC_VER_MINOR__) "-fmadon-ex2approxftz-nrl-" NRL_SRC_HASH;
}

extern "C" uint64_t nrl_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" const char* nrl_error_string(int code) {
    switch (code) {
        case NRL_OK: return "success";
        case NRL_E_BAD_ARG: return "nrl: bad argument (null pointer, zero size, struct size mismatch or misaligned pointer)";
        case NRL_E_UNSUPPORTED: return "nrl: unsupported dtype or option";
        case NRL_E_WORKSPACE: return "nrl: scratch buffer missing or too small (for nrl_row_fwd_static: the shape needs more than the fixed NRL_STATIC_SCRATCH_BYTES)";
        case NRL_E_ROW_STATUS: return "nrl: a row has no allowed token (every logit -inf) or a NaN";
        case NRL_E_NO_DEVICE: return "nrl: no CUDA device or no current context";
        case NRL_E_NOT_FINITE: return "nrl: a scored log-probability is not finite";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "nrl: unknown error";
    }
}

// The row kernels are compiled twice, once per mask format: here for a byte per token (and for
// calls without a mask), in nrl_bits.cu for a bit per token.
#define NRL_ROW_FWD_ENTRY nrl_row_fwd_bytes
#define NRL_ROW_BWD_ENTRY nrl_row_bwd_bytes
#include "row_api.inl"
int nrl_row_fwd_bits(const nrl_row_fwd_args* a, nrl_stream stream);
int nrl_row_bwd_bits(const nrl_row_bwd_args* a, nrl_stream stream);

extern "C" int nrl_row_fwd(const nrl_row_fwd_args* a, nrl_stream stream) {
    if (a && a->struct_size == sizeof(nrl_row_fwd_args) && (a->flags & NRL_FWD_MASK_BITS)) return nrl_row_fwd_bits(a, stream);
    return nrl_row_fwd_bytes(a, stream);
}

extern "C" int nrl_row_bwd(const nrl_row_bwd_args* a, nrl_stream stream) {
    if (a && a->struct_size == sizeof(nrl_row_bwd_args) && a->mask_bits) return nrl_row_bwd_bits(a, stream);
    return nrl_row_bwd_bytes(a, stream);
}

extern "C" uint64_t nrl_row_fwd_workspace_bytes(uint64_t rows, uint32_t V) {
    if (rows == 0 || V == 0) return 0;
    uint32_t ns = fwd_nsplit(rows, V);
    return ns == 1 ? 0 : rows * ns * kWarps * kPartFloats * sizeof(float);
}

// ---- forward without a caller-provided workspace -------------------------------------------------
//
// For callers that may not allocate device memory (see include/nrl.h). The scratch of the split
// forward lives in this array, inside the library's device image, once per GPU that loads it.
static __device__ __align__(256) unsigned char g_static_scratch[NRL_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the
// address is looked up once per device with that device current, and that pointer goes to the
// kernels.
static const int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices];
static std::mutex g_static_scratch_lock;

static int static_scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return NRL_E_NO_DEVICE;
    std::lock_guard<std::mutex> hold(g_static_scratch_lock);
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return NRL_E_NO_DEVICE;
        g_static_scratch_addr[dev] = p;
    }
    *out = g_static_scratch_addr[dev];
    return NRL_OK;
}

extern "C" int nrl_row_fwd_static(const nrl_row_fwd_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_row_fwd_args)) return NRL_E_BAD_ARG;
    if (nrl_row_fwd_workspace_bytes(a->rows, a->V) > NRL_STATIC_SCRATCH_BYTES) return NRL_E_WORKSPACE;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc) return rc;
    nrl_row_fwd_args b = *a;
    b.workspace = (nrl_devptr)(uintptr_t)scratch;
    b.workspace_bytes = NRL_STATIC_SCRATCH_BYTES;
    return nrl_row_fwd(&b, stream);
}

// ---- token-level ---------------------------------------------------------------------------------

static int fill_tok(TokParams& p, const nrl_token_loss_args* a) {
    if (!a || a->struct_size != sizeof(nrl_token_loss_args)) return NRL_E_BAD_ARG;
    if (a->S == 0 || a->B == 0 || a->T == 0 || !a->logp) return NRL_E_BAD_ARG;
    if (a->kind > NRL_LOSS_K3) return NRL_E_UNSUPPORTED;
    bool needs_w = a->kind == NRL_LOSS_PG || a->kind == NRL_LOSS_PPO;
    bool needs_o = a->kind != NRL_LOSS_PG;
    if ((needs_w && !a->weights) || (needs_o && !a->other)) return NRL_E_BAD_ARG;
    if (a->kind == NRL_LOSS_PPO) {
        // Clip::check (src/nn/rl.rs:189-197)
        if (!(a->clip_low >= 0.0 && a->clip_low < 1.0 && a->clip_high >= 0.0) || !isfinite(a->clip_low) || !isfinite(a->clip_high)) return NRL_E_BAD_ARG;
        if (a->has_dual && !(a->dual > 1.0 && isfinite(a->dual))) return NRL_E_BAD_ARG;
    }
    if (a->has_clamp && !(a->clamp > 0.0)) return NRL_E_BAD_ARG;
    memset(&p, 0, sizeof p);
    p.logp = (const float*)a->logp;
    p.other = (const float*)a->other;
    p.weights = (const float*)a->weights;
    p.mask = (const float*)a->mask;
    p.loss = (float*)a->loss;
    p.upstream = (const float*)a->upstream;
    p.dloss = (float*)a->dloss_dlogp;
    p.n = a->S * a->B * a->T;
    p.T = a->T;
    p.kind = a->kind;
    p.w_per_seq = a->weights_per_sequence;
    p.has_dual = a->has_dual;
    p.has_clamp = a->has_clamp;
    p.accumulate = a->accumulate ? 1u : 0u;
    p.ratio_lo = (float)(1.0 - a->clip_low);
    p.ratio_hi = (float)(1.0 + a->clip_high);
    p.neg_dual = (float)(-a->dual);
    p.clamp = (float)a->clamp;
    return NRL_OK;
}

extern "C" int nrl_token_loss(const nrl_token_loss_args* a, nrl_stream stream) {
    TokParams p;
    int rc = fill_tok(p, a);
    if (rc) return rc;
    uint64_t blocks = (p.n + 255) / 256;
    if (blocks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    token_loss_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return after_launch();
}

extern "C" int nrl_token_objective(const nrl_token_objective_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_token_objective_args)) return NRL_E_BAD_ARG;
    ObjectiveParams p;
    memset(&p, 0, sizeof p);
    int rc = fill_tok(p.tok, &a->policy);
    if (rc) return rc;
    if (a->reduction != NRL_REDUCE_SUM && a->reduction != NRL_REDUCE_TOKEN_MEAN && a->reduction != NRL_REDUCE_SEQUENCE_MEAN) return NRL_E_UNSUPPORTED;
    if (a->policy.S > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    if ((a->g_kl && !a->kl) || (a->g_ent && !a->entropy)) return NRL_E_BAD_ARG;
    p.tok.loss = nullptr;
    p.tok.upstream = nullptr;
    p.tok.dloss = nullptr;
    p.kl = (const float*)a->kl;
    p.entropy = (const float*)a->entropy;
    p.up_policy = (const float*)a->up_policy;
    p.up_kl = (const float*)a->up_kl;
    p.up_entropy = (const float*)a->up_entropy;
    p.out_policy = (float*)a->out_policy;
    p.out_kl = (float*)a->out_kl;
    p.out_entropy = (float*)a->out_entropy;
    p.g_logp = (float*)a->g_logp;
    p.g_kl = (float*)a->g_kl;
    p.g_ent = (float*)a->g_ent;
    p.B = a->policy.B;
    p.T = a->policy.T;
    p.reduction = a->reduction;
    token_objective_kernel<<<(unsigned)a->policy.S, kFoldThreads, 0, (cudaStream_t)stream>>>(p);
    return after_launch();
}

extern "C" int nrl_clip_fraction(const nrl_token_loss_args* a, nrl_devptr out, nrl_stream stream) {
    TokParams p;
    int rc = fill_tok(p, a);
    if (rc) return rc;
    if (a->kind != NRL_LOSS_PPO || !out) return NRL_E_BAD_ARG;
    if (a->S > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    clip_fraction_kernel<<<(unsigned)a->S, kRedThreads, 0, (cudaStream_t)stream>>>(p, a->B * a->T, (float*)out);
    return after_launch();
}

extern "C" int nrl_reduce_tokens(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, nrl_devptr per, nrl_devptr mask, nrl_devptr out, nrl_stream stream) {
    if (S == 0 || B == 0 || T == 0 || !per || !out || reduction > NRL_REDUCE_SEQUENCE_MEAN) return NRL_E_BAD_ARG;
    if (reduction == NRL_REDUCE_NONE) {
        if (per == out) return NRL_OK;
        return cuda_rc(cudaMemcpyAsync((void*)out, (const void*)per, S * B * T * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    }
    if (S > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    reduce_tokens_kernel<<<(unsigned)S, kFoldThreads, 0, (cudaStream_t)stream>>>(reduction, B, T, (const float*)per, (const float*)mask, (float*)out);
    return after_launch();
}

extern "C" int nrl_reduce_tokens_partial(uint64_t n_seq, uint64_t T, nrl_devptr per, nrl_devptr mask, nrl_devptr pairs, nrl_stream stream) {
    if (n_seq == 0 || T == 0 || !per || !pairs || (pairs & 7u) || ((per | mask) & 3u)) return NRL_E_BAD_ARG;
    const uint64_t blocks = (n_seq + 7) / 8;
    if (blocks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    seq_pairs_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(n_seq, T, (const float*)per, (const float*)mask, (float2*)pairs);
    return after_launch();
}

extern "C" int nrl_reduce_tokens_fold(uint32_t reduction, uint64_t S, uint64_t B, nrl_devptr pairs, nrl_devptr out, nrl_stream stream) {
    if (S == 0 || B == 0 || !pairs || !out || (pairs & 7u) || (out & 3u)) return NRL_E_BAD_ARG;
    if (reduction == NRL_REDUCE_NONE || reduction > NRL_REDUCE_SEQUENCE_MEAN) return NRL_E_BAD_ARG;
    const uint64_t n = reduction == NRL_REDUCE_PER_SEQUENCE ? S * B : S;
    const uint64_t blocks = (n + 127) / 128;
    if (blocks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    fold_pairs_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(reduction, S, B, (const float2*)pairs, (float*)out);
    return after_launch();
}

extern "C" int nrl_reduce_tokens_bwd_pairs(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, uint64_t seq_begin, uint64_t n_seq, nrl_devptr pairs, nrl_devptr mask,
                                           nrl_devptr g_out, nrl_devptr d_per, nrl_stream stream) {
    if (S == 0 || B == 0 || T == 0 || n_seq == 0 || !g_out || !d_per || reduction > NRL_REDUCE_SEQUENCE_MEAN) return NRL_E_BAD_ARG;
    if (seq_begin + n_seq > S * B || (reduction != NRL_REDUCE_NONE && (!pairs || (pairs & 7u)))) return NRL_E_BAD_ARG;
    const uint64_t blocks = (n_seq + 7) / 8;
    if (blocks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    reduce_tokens_bwd_pairs_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(reduction, B, T, seq_begin, n_seq, (const float2*)pairs, (const float*)mask, (const float*)g_out,
                                                                                  (float*)d_per);
    return after_launch();
}

extern "C" int nrl_reduce_tokens_bwd(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, nrl_devptr mask, nrl_devptr g_out, nrl_devptr d_per, nrl_stream stream) {
    if (S == 0 || B == 0 || T == 0 || !g_out || !d_per || reduction > NRL_REDUCE_SEQUENCE_MEAN) return NRL_E_BAD_ARG;
    if (S > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    reduce_tokens_bwd_kernel<<<(unsigned)S, kFoldThreads, 0, (cudaStream_t)stream>>>(reduction, B, T, (const float*)mask, (const float*)g_out, (float*)d_per);
    return after_launch();
}

extern "C" int nrl_mask_rows(uint64_t n, nrl_devptr x, nrl_devptr mask, nrl_devptr out, nrl_stream stream) {
    if (n == 0 || !x || !out) return NRL_E_BAD_ARG;
    if ((n + 255) / 256 > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    mask_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, (const float*)x, (const float*)mask, (float*)out);
    return after_launch();
}

extern "C" int nrl_group_advantages(uint64_t groups, uint32_t n, uint32_t norm_std, double eps, uint32_t unbiased, nrl_devptr rewards, nrl_devptr out, nrl_stream stream) {
    if (groups == 0 || n == 0 || !rewards || !out || ((rewards | out) & 3u)) return NRL_E_BAD_ARG;
    if (norm_std && (!(eps >= 0.0) || (unbiased && n < 2))) return NRL_E_BAD_ARG;
    if ((groups + 127) / 128 > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    group_advantages_kernel<<<(unsigned)((groups + 127) / 128), 128, 0, (cudaStream_t)stream>>>(groups, n, norm_std != 0, eps, unbiased != 0, (const float*)rewards, (float*)out);
    return after_launch();
}

// ---- cross-entropy family -------------------------------------------------------------------------

extern "C" int nrl_row_sum(uint32_t dtype, uint64_t rows, uint32_t V, nrl_devptr logits, nrl_devptr out, nrl_stream stream) {
    if (rows == 0 || V == 0 || !logits || !out) return NRL_E_BAD_ARG;
    if (dtype != NRL_F32 && dtype != NRL_BF16) return NRL_E_UNSUPPORTED;
    if ((logits & (dtype == NRL_F32 ? 3u : 1u)) || (out & 3u)) return NRL_E_BAD_ARG;
    if (rows > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    const bool vec = V % kVec == 0 && (logits & 15u) == 0;
    if (dtype == NRL_F32) row_sum_kernel<NRL_F32><<<(unsigned)rows, kSumThreads, 0, (cudaStream_t)stream>>>((const void*)logits, V, vec, (float*)out);
    else row_sum_kernel<NRL_BF16><<<(unsigned)rows, kSumThreads, 0, (cudaStream_t)stream>>>((const void*)logits, V, vec, (float*)out);
    return after_launch();
}

extern "C" int nrl_ce_tokens(const nrl_ce_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_ce_args)) return NRL_E_BAD_ARG;
    if (a->n == 0 || a->V == 0 || !a->logp) return NRL_E_BAD_ARG;
    if (!(a->smoothing >= 0.0 && a->smoothing <= 1.0)) return NRL_E_BAD_ARG;  // "label smoothing outside [0, 1]"
    if (!a->loss && !a->upstream) return NRL_E_BAD_ARG;
    if (a->upstream && !a->g_logp) return NRL_E_BAD_ARG;
    if (a->smoothing > 0.0 && (!a->rowstats || (a->rowstats & 15u) || !a->logit_sum || (a->upstream && !a->g_uniform))) return NRL_E_BAD_ARG;
    CeParams p;
    memset(&p, 0, sizeof p);
    p.logp = (const float*)a->logp;
    p.rowstats = (const float*)a->rowstats;
    p.logit_sum = (const float*)a->logit_sum;
    p.keep = (const float*)a->keep;
    p.upstream = (const float*)a->upstream;
    p.loss = (float*)a->loss;
    p.g_logp = (float*)a->g_logp;
    p.g_uniform = a->smoothing > 0.0 ? (float*)a->g_uniform : nullptr;
    p.n = a->n;
    p.eps = (float)a->smoothing;
    p.one_minus_eps = (float)(1.0 - a->smoothing);
    p.inv_v = 1.0f / (float)a->V;
    uint64_t blocks = (p.n + 255) / 256;
    if (blocks > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    ce_tokens_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return after_launch();
}

// ---- the reference's Gumbel-max sampler ------------------------------------------------------------

extern "C" int nrl_sample_gumbel(const nrl_gumbel_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_gumbel_args)) return NRL_E_BAD_ARG;
    GumbelParams p;
    memset(&p, 0, sizeof p);
    int rc = fill_fwd_params(p.in, a->dtype, a->V, a->rows, a->temperature, a->logits, 0, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    if (rc) return rc;
    if (!a->tokens || (a->tokens & 3u)) return NRL_E_BAD_ARG;
    if (a->rows > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    for (int i = 0; i < 8; i++)
        p.key[i] = (uint32_t)a->seed[4 * i] | (uint32_t)a->seed[4 * i + 1] << 8 | (uint32_t)a->seed[4 * i + 2] << 16 | (uint32_t)a->seed[4 * i + 3] << 24;
    p.word_offset = a->word_offset;
    p.tokens = (int32_t*)a->tokens;
    p.status = (uint8_t*)a->status;
    const bool vec = can_vectorise(a->V, a->logits, 0, a->allow_mask, a->allow_row_stride, a->add_mask, a->add_row_stride);
    const unsigned grid = (unsigned)a->rows;
    cudaStream_t st = (cudaStream_t)stream;
#define NRL_GUMBEL(DT)                                                                                               \
    do {                                                                                                             \
        if (a->allow_mask) { if (vec) gumbel_argmax_kernel<DT, true, true><<<grid, kGumbelThreads, 0, st>>>(p); else gumbel_argmax_kernel<DT, true, false><<<grid, kGumbelThreads, 0, st>>>(p); } \
        else               { if (vec) gumbel_argmax_kernel<DT, false, true><<<grid, kGumbelThreads, 0, st>>>(p); else gumbel_argmax_kernel<DT, false, false><<<grid, kGumbelThreads, 0, st>>>(p); } \
    } while (0)
    if (a->dtype == NRL_F32) NRL_GUMBEL(NRL_F32);
    else NRL_GUMBEL(NRL_BF16);
#undef NRL_GUMBEL
    return after_launch();
}

// ---- generic lane reductions ---------------------------------------------------------------------

template <int DT>
static void launch_lane(const nrl_lane_args* a, bool vec, unsigned grid, unsigned threads, cudaStream_t st) {
    const void* x = (const void*)a->x;
    float* out = (float*)a->out;
    switch (a->op) {
        case NRL_LANE_SOFTMAX:
            if (vec) lane_softmax_kernel<DT, true, false><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            else lane_softmax_kernel<DT, false, false><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            break;
        case NRL_LANE_LOG_SOFTMAX:
            if (vec) lane_softmax_kernel<DT, true, true><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            else lane_softmax_kernel<DT, false, true><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            break;
        case NRL_LANE_LOGSUMEXP:
            if (vec) lane_logsumexp_kernel<DT, true><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            else lane_logsumexp_kernel<DT, false><<<grid, threads, 0, st>>>(x, out, a->rows, a->V);
            break;
        case NRL_LANE_ARGMAX:
            if (vec) lane_argmax_kernel<DT, true><<<grid, threads, 0, st>>>(x, (int32_t*)a->out_index, out, a->rows, a->V);
            else lane_argmax_kernel<DT, false><<<grid, threads, 0, st>>>(x, (int32_t*)a->out_index, out, a->rows, a->V);
            break;
        case NRL_LANE_SUM: {
            // eight lanes per row: few rows run small blocks so that every SM gets some
            const unsigned bt = a->rows >= 148ull * 8 * 32 ? kLaneThreads : 64;
            const uint64_t blocks = (a->rows + bt / 8 - 1) / (bt / 8);
            lane_sum_ordered_kernel<DT><<<(unsigned)(blocks < 148ull * 32 ? blocks : 148ull * 32), bt, 0, st>>>(x, out, a->rows, a->V);
            break;
        }
        case NRL_LANE_LOGSUMEXP_BWD:
            if (vec) lane_logsumexp_bwd_kernel<DT, true><<<grid, threads, 0, st>>>(x, (const float*)a->lse, (const float*)a->g, out, a->rows, a->V);
            else lane_logsumexp_bwd_kernel<DT, false><<<grid, threads, 0, st>>>(x, (const float*)a->lse, (const float*)a->g, out, a->rows, a->V);
            break;
        default: break;
    }
}

// softmax / log_softmax on clusters of `csize` CTAs, each holding `per` vectors of a row
template <int DT, bool LOG>
static int launch_lane_cluster_as(const nrl_lane_args* a, uint32_t csize, uint32_t per, uint32_t vec_bytes, cudaStream_t st) {
    auto kernel = lane_softmax_cluster_kernel<DT, LOG>;
    const uint32_t smem = per * vec_bytes;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(csize, 1, 1);
    cfg.blockDim = dim3(kLaneClusterThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // how many clusters of this shape the device holds at once: asked once per (device, shape) and kernel
    static std::atomic<uint64_t> known{0};  // device << 56 | cluster size << 48 | shared memory << 16 | resident clusters
    int dev = 0, resident = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    const uint64_t key = ((uint64_t)(dev & 0xff) << 56) | ((uint64_t)csize << 48) | ((uint64_t)smem << 16);
    const uint64_t seen = known.load(std::memory_order_relaxed);
    if ((seen & ~0xffffull) == key && (seen & 0xffffull) != 0) {
        resident = (int)(seen & 0xffffull);
    } else {
        e = cudaOccupancyMaxActiveClusters(&resident, kernel, &cfg);
        if (e != cudaSuccess || resident < 1) {
            (void)cudaGetLastError();
            return NRL_E_UNSUPPORTED;  // the caller falls back to the kernel that reads the row twice
        }
        known.store(key | (uint64_t)(resident > 0xffff ? 0xffff : resident), std::memory_order_relaxed);
    }
    const uint64_t clusters = a->rows < (uint64_t)resident ? a->rows : (uint64_t)resident;
    cfg.gridDim = dim3((unsigned)(clusters * csize), 1, 1);
    e = cudaLaunchKernelEx(&cfg, kernel, (const void*)a->x, (float*)a->out, (uint64_t)a->rows, (uint32_t)a->V, per);
    if (e != cudaSuccess) return (int)e;
    return after_launch();
}

static int launch_lane_cluster(const nrl_lane_args* a, uint32_t csize, uint32_t per, uint32_t vec_bytes, cudaStream_t st) {
    const bool log = a->op == NRL_LANE_LOG_SOFTMAX;
    if (a->dtype == NRL_F32) return log ? launch_lane_cluster_as<NRL_F32, true>(a, csize, per, vec_bytes, st) : launch_lane_cluster_as<NRL_F32, false>(a, csize, per, vec_bytes, st);
    return log ? launch_lane_cluster_as<NRL_BF16, true>(a, csize, per, vec_bytes, st) : launch_lane_cluster_as<NRL_BF16, false>(a, csize, per, vec_bytes, st);
}

extern "C" int nrl_lane_op(const nrl_lane_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_lane_args)) return NRL_E_BAD_ARG;
    if (a->rows == 0 || a->V == 0 || !a->x || a->op > NRL_LANE_LOGSUMEXP_BWD) return NRL_E_BAD_ARG;
    if (a->dtype != NRL_F32 && a->dtype != NRL_BF16) return NRL_E_UNSUPPORTED;
    const bool bwd_y = a->op == NRL_LANE_SOFTMAX_BWD || a->op == NRL_LANE_LOG_SOFTMAX_BWD;
    if (bwd_y && a->dtype != NRL_F32) return NRL_E_UNSUPPORTED;
    if (a->op == NRL_LANE_ARGMAX ? !a->out_index : !a->out) return NRL_E_BAD_ARG;
    if ((bwd_y || a->op == NRL_LANE_LOGSUMEXP_BWD) && !a->g) return NRL_E_BAD_ARG;
    if (a->op == NRL_LANE_LOGSUMEXP_BWD && !a->lse) return NRL_E_BAD_ARG;
    const uint64_t esize = a->dtype == NRL_F32 ? 4 : 2;
    if ((a->x & (esize - 1)) || (a->out & 3u) || (a->out_index & 3u) || (a->g & 3u) || (a->lse & 3u)) return NRL_E_BAD_ARG;
    const bool vec = a->V % kVec == 0 && aligned16(a->x) && aligned16(a->out) && (!bwd_y || aligned16(a->g));
    // The backward rules read two [rows, V] inputs twice: when the rows that 8 blocks of 256 threads
    // per SM would hold in flight outgrow L2, one block of 1024 threads per SM runs instead
    // (measured: +8 % there). The forward softmax of such rows runs on clusters (below); on this
    // kernel it is faster with the many small blocks.
    const uint64_t row_bytes = (uint64_t)a->V * esize * 2;
    const bool fwd_full = a->op == NRL_LANE_SOFTMAX || a->op == NRL_LANE_LOG_SOFTMAX;
    const bool wide = bwd_y && row_bytes * 1184ull > (96ull << 20);
    const unsigned threads = wide ? kLaneMaxThreads : kLaneThreads;
    const uint64_t cap = wide ? 148ull : 148ull * 8ull;
    const unsigned grid = (unsigned)(a->rows < cap ? a->rows : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (fwd_full && vec && row_bytes * 1184ull > (96ull << 20)) {
        // rows that L2 would not keep until their second read: a cluster holds the row in shared memory
        const uint32_t nvec = a->V / kVec, vec_bytes = (uint32_t)(kVec * esize);
        uint32_t csize = (uint32_t)(((uint64_t)nvec * vec_bytes + kLaneSliceBytes - 1) / kLaneSliceBytes);
        while (csize <= kLaneMaxCluster && (uint64_t)((nvec + csize - 1) / csize) * vec_bytes > kLaneSliceBytes) csize++;
        // a little longer (V = 151 936 f32 needs 74.2 KB per CTA of 8): the largest cluster with two CTAs per SM
        if (csize > kLaneMaxCluster && (uint64_t)((nvec + kLaneMaxCluster - 1) / kLaneMaxCluster) * vec_bytes <= kLaneSliceBytesTwo) csize = kLaneMaxCluster;
        if (csize <= kLaneMaxCluster) {
            const int rc = launch_lane_cluster(a, csize, (nvec + csize - 1) / csize, vec_bytes, st);
            if (rc != NRL_E_UNSUPPORTED) return rc;
        }
    }
    if (bwd_y) {
        const float *y = (const float*)a->x, *g = (const float*)a->g;
        float* dx = (float*)a->out;
        if (a->op == NRL_LANE_SOFTMAX_BWD) {
            if (vec) lane_softmax_bwd_kernel<true, false><<<grid, threads, 0, st>>>(y, g, dx, a->rows, a->V);
            else lane_softmax_bwd_kernel<false, false><<<grid, threads, 0, st>>>(y, g, dx, a->rows, a->V);
        } else {
            if (vec) lane_softmax_bwd_kernel<true, true><<<grid, threads, 0, st>>>(y, g, dx, a->rows, a->V);
            else lane_softmax_bwd_kernel<false, true><<<grid, threads, 0, st>>>(y, g, dx, a->rows, a->V);
        }
    } else if (a->dtype == NRL_F32) {
        launch_lane<NRL_F32>(a, vec, grid, threads, st);
    } else {
        launch_lane<NRL_BF16>(a, vec, grid, threads, st);
    }
    return after_launch();
}

// ---- host-resident rows --------------------------------------------------------------------------

extern "C" int nrl_host_pack(nrl_pack_args* a) {
    if (!a || a->struct_size != sizeof(nrl_pack_args)) return NRL_E_BAD_ARG;
    if (a->rows == 0 || a->V == 0 || a->V % kVec != 0 || a->V > 262144u) return NRL_E_BAD_ARG;
    if (!a->logits || !a->allow_mask || !a->live_words || !a->row_offset || !a->packed_logits || !a->packed_mask) return NRL_E_BAD_ARG;
    if ((a->ref_logits != nullptr) != (a->packed_ref != nullptr)) return NRL_E_BAD_ARG;
    if (a->dtype == NRL_BF16) return a->ref_logits ? host_pack_impl<2, true>(a) : host_pack_impl<2, false>(a);
    if (a->dtype == NRL_F32) return a->ref_logits ? host_pack_impl<4, true>(a) : host_pack_impl<4, false>(a);
    return NRL_E_UNSUPPORTED;
}

extern "C" int nrl_host_pack_bits(uint64_t rows, uint32_t V, const uint8_t* allow_mask, uint32_t* bits, uint32_t threads) {
    if (rows == 0 || V == 0 || !allow_mask || !bits) return NRL_E_BAD_ARG;
    return host_pack_bits_impl(rows, V, allow_mask, bits, threads);
}

extern "C" int nrl_unpack_rows(const nrl_unpack_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_unpack_args)) return NRL_E_BAD_ARG;
    if (a->rows == 0 || a->V == 0 || a->V % kVec != 0 || a->V > 262144u || a->rows > 0x7fffffffull) return NRL_E_BAD_ARG;
    if (!a->live_words || !a->row_offset || !a->packed_logits || !a->packed_mask || !a->logits || !a->allow_mask) return NRL_E_BAD_ARG;
    if ((a->ref_logits != 0) != (a->packed_ref != 0)) return NRL_E_BAD_ARG;
    if ((a->logits | a->ref_logits | a->allow_mask | a->packed_logits | a->packed_ref) & 15u) return NRL_E_BAD_ARG;
    if ((a->packed_mask | a->live_words) & 7u) return NRL_E_BAD_ARG;
    const unsigned grid = (unsigned)a->rows;
    cudaStream_t st = (cudaStream_t)stream;
#define NRL_UNPACK(ES, RF) unpack_rows_kernel<ES, RF><<<grid, 256, 0, st>>>(a->V, (const uint64_t*)a->live_words, (const uint32_t*)a->row_offset, (const uint4*)a->packed_logits, \
                                                                          (const uint4*)a->packed_ref, (const uint2*)a->packed_mask, (char*)a->logits, (char*)a->ref_logits, (uint8_t*)a->allow_mask)
    if (a->dtype == NRL_BF16) { if (a->ref_logits) NRL_UNPACK(2, true); else NRL_UNPACK(2, false); }
    else if (a->dtype == NRL_F32) { if (a->ref_logits) NRL_UNPACK(4, true); else NRL_UNPACK(4, false); }
    else return NRL_E_UNSUPPORTED;
#undef NRL_UNPACK
    return after_launch();
}

extern "C" int nrl_expand_bitmask(uint64_t rows, uint32_t V, nrl_devptr bits, uint64_t bits_row_stride_words, nrl_devptr allow_mask, nrl_stream stream) {
    if (rows == 0 || V == 0 || !bits || !allow_mask || (bits & 3u)) return NRL_E_BAD_ARG;
    const uint32_t words = (V + 31) / 32;
    if (bits_row_stride_words != 0 && bits_row_stride_words < words) return NRL_E_BAD_ARG;
    const uint64_t total = rows * (uint64_t)((V + 7) / 8);
    const uint64_t blocks = (total + 255) / 256;
    expand_bitmask_kernel<<<(unsigned)(blocks < 148ull * 32 ? blocks : 148ull * 32), 256, 0, (cudaStream_t)stream>>>(rows, V, words, bits_row_stride_words, (const uint32_t*)bits, (uint8_t*)allow_mask);
    return after_launch();
}

extern "C" int nrl_check_status(nrl_devptr status, uint64_t rows, nrl_stream stream, uint64_t* first_bad_row, uint32_t* bits) {
    if (!status || rows == 0) return NRL_E_BAD_ARG;
    // read back in pieces of a fixed size: no host allocation that could fail
    static const uint64_t kPiece = 1u << 15;
    uint8_t host[kPiece];
    for (uint64_t r0 = 0; r0 < rows; r0 += kPiece) {
        const uint64_t n = rows - r0 < kPiece ? rows - r0 : kPiece;
        cudaError_t e = cudaMemcpyAsync(host, (const void*)(status + r0), n, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
        for (uint64_t i = 0; i < n; i++)
            if (host[i]) {
                if (first_bad_row) *first_bad_row = r0 + i;
                if (bits) *bits = host[i];
                return NRL_E_ROW_STATUS;
            }
    }
    return NRL_OK;
}

extern "C" int nrl_check_scored_finite(nrl_devptr logp, nrl_devptr mask, uint64_t n, nrl_devptr result, nrl_stream stream, uint64_t* first_position, float* value) {
    if (!logp || n == 0 || !result || (result & 7u) || ((logp | mask) & 3u)) return NRL_E_BAD_ARG;
    first_nonfinite_kernel<<<1, kScanThreads, 0, (cudaStream_t)stream>>>(n, (const float*)logp, (const float*)mask, (uint64_t*)result);
    int rc = after_launch();
    if (rc) return rc;
    uint64_t host[2] = {~0ull, 0ull};
    cudaError_t e = cudaMemcpyAsync(host, (const void*)result, sizeof host, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    if (host[0] == ~0ull) return NRL_OK;
    if (first_position) *first_position = host[0];
    if (value) {
        const uint32_t b = (uint32_t)host[1];
        memcpy(value, &b, sizeof b);
    }
    return NRL_E_NOT_FINITE;
}

// ---- readout-fused row statistics (tcgen05) ---------------------------------------------------------

// Column ranges per row block. Work is laid out in groups: a group is some row blocks times every
// column range, at most one wave of CTAs (148) or CTA pairs (74), and runs as one wave, so that the
// group's hidden states (rows · d · 2 bytes) stay in L2 while its CTAs walk the vocabulary and each W
// tile is fetched once per group. Measured on B200 at d = 4096: 18 944 rows reach 0.82 PFLOP/s
// with one range (148 MB of hidden states in flight) and 1.24 with four (37 MB). The count taken
// (at most 16, each range at least 8 tiles) is the one that fills the waves best among those whose
// group keeps at most 40 MB of hidden states in flight. A function of (rows, V, d) only.
static uint32_t readout_nsplit(uint64_t rows, uint32_t V, uint32_t d, bool pairs) {
    // the unit is a CTA (128 rows, 148 per wave) or a CTA pair (256 rows, 74 per wave)
    const uint64_t unit_rows = pairs ? 2 * kRoBM : kRoBM, wave = pairs ? 74 : 148;
    const uint64_t rb = (rows + unit_rows - 1) / unit_rows;
    const uint32_t tiles = (V + kRoBN - 1) / kRoBN;
    const uint64_t block_bytes = unit_rows * d * 2;
    uint32_t best = 0;
    double best_eff = -1.0;
    for (int pass = 0; pass < 2 && !best; pass++) {  // second pass: no count meets the footprint, take the best anyway
        for (uint32_t s = 1; s <= 16 && (s == 1 || tiles / s >= 8); s++) {
            uint64_t gb = wave / s;
            if (gb < 1) gb = 1;
            if (gb > rb) gb = rb;
            if (pass == 0 && gb * block_bytes > (40ull << 20)) continue;
            const uint64_t ctas = rb * s;
            const double eff = (double)ctas / (double)(wave * ((ctas + wave - 1) / wave));
            if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
        }
    }
    return best ? best : 1;
}

static uint64_t readout_parts_bytes(uint64_t rows, uint32_t V, uint32_t d) {
    const uint32_t a = readout_nsplit(rows, V, d, false), b = readout_nsplit(rows, V, d, true);
    return (rows * (a > b ? a : b) * kRoPartFloats * sizeof(float) + 255) & ~255ull;
}

// Rows per launch. Every CTA of a launch has the same amount of work and the CTAs that walk one column range share its W
// tiles through L2 only while they stay in step; over tens of waves they drift apart (B200, d = 4096, V = 128 256: 1.34
// PFLOP/s at 65 536 rows, 1.24 at 131 072, 1.13 at 262 144 in one launch). So a large batch goes out as launches of 8192 to
// 24 576 rows, each on CTA pairs and each a whole number of full waves: the count of 256-row blocks b that wastes the
// fewest of its waves' 74 pair slots, the larger b on a tie.
static uint64_t readout_chunk_rows(uint64_t rows, uint32_t V, uint32_t d, uint32_t flags) {
    if ((flags & NRL_READOUT_ONE_CTA) || rows <= 24576) return rows;
    uint64_t best = 64;
    double best_eff = -1.0;
    for (uint64_t b = 32; b <= 96; b++) {
        const uint32_t s = readout_nsplit(b * 2 * kRoBM, V, d, true);
        uint64_t gb = 74 / s;
        if (gb < 1) gb = 1;
        if (gb > b) gb = b;
        const uint64_t slots = ((b + gb - 1) / gb * gb * s + 73) / 74 * 74;  // the launch pads its last group
        const double eff = (double)(b * s) / (double)slots;
        if (eff >= best_eff) { best_eff = eff; best = b; }
    }
    return best * 2 * kRoBM;
}

static uint64_t readout_workspace_one(uint64_t rows, uint32_t V, uint32_t d, uint32_t flags);

extern "C" uint64_t nrl_readout_workspace_bytes(uint64_t rows, uint32_t V, uint32_t d, uint32_t flags) {
    if (rows == 0 || V == 0 || d == 0) return 0;
    const uint64_t chunk = readout_chunk_rows(rows, V, d, flags);
    if (chunk >= rows) return readout_workspace_one(rows, V, d, flags);
    const uint64_t a = readout_workspace_one(chunk, V, d, flags), tail = rows % chunk;
    const uint64_t b = tail ? readout_workspace_one(tail, V, d, flags) : 0;
    return a > b ? a : b;
}

static uint64_t readout_workspace_one(uint64_t rows, uint32_t V, uint32_t d, uint32_t flags) {
    uint64_t n = readout_parts_bytes(rows, V, d);
    if (flags & NRL_READOUT_SAMPLE) {
        const uint64_t nslabs = (uint64_t)((V + kRoBN - 1) / kRoBN) * (kRoBN / kRoLogCols);
        n += (rows * nslabs * sizeof(float2) + 255) & ~255ull;      // the mass log
        n += (rows * sizeof(ReadoutPick) + 255) & ~255ull;          // each row's slab and residual
        n += ((nslabs + 1) * sizeof(uint32_t) + 255) & ~255ull;     // rows grouped by slab: starts
        n += (rows * sizeof(uint32_t) + 255) & ~255ull;             //                       and order
    }
    return n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: the library links no libcuda.
static int encode_bf16_2d(CUtensorMap* map, uint64_t base, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
    static std::atomic<void*> fn{nullptr};
    void* f = fn.load(std::memory_order_acquire);
    if (!f) {
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q);
        if (e != cudaSuccess) return (int)e;
        if (q != cudaDriverEntryPointSuccess || !f) return NRL_E_UNSUPPORTED;
        fn.store(f, std::memory_order_release);
    }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * 2};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)f)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NRL_OK : NRL_E_BAD_ARG;
}

static int readout_fwd_one(const nrl_readout_args* a, nrl_stream stream);

extern "C" int nrl_readout_fwd(const nrl_readout_args* a, nrl_stream stream) {
    if (!a || a->struct_size != sizeof(nrl_readout_args)) return NRL_E_BAD_ARG;
    if (a->rows == 0 || a->V == 0 || a->d == 0 || !a->hidden || !a->weights) return NRL_E_BAD_ARG;
    if (a->flags & ~(uint32_t)(NRL_READOUT_W_VD | NRL_READOUT_ROUND_BF16 | NRL_READOUT_ONE_CTA | NRL_READOUT_SAMPLE | NRL_READOUT_GREEDY | NRL_READOUT_MASK_BITS)) return NRL_E_BAD_ARG;
    // TMA wants 16-byte aligned bases and row pitches
    if (a->V % 8 != 0 || a->d % 8 != 0 || ((a->hidden | a->weights) & 15u)) return NRL_E_UNSUPPORTED;
    if ((a->tokens & 3u) || (a->logp & 3u) || (a->entropy & 3u) || (a->rowstats & 15u) || (a->logits_out & 3u) || (a->workspace & 15u)) return NRL_E_BAD_ARG;
    if (a->logp && !a->tokens) return NRL_E_BAD_ARG;
    const bool sample = (a->flags & NRL_READOUT_SAMPLE) != 0;
    if (sample && (!a->uniforms || (a->uniforms & 3u) || !a->tokens)) return NRL_E_BAD_ARG;
    if ((a->flags & NRL_READOUT_GREEDY) && (sample || !a->tokens)) return NRL_E_BAD_ARG;
    if (a->reserved != 0 || !(a->temperature >= 0.f) || !isfinite(a->temperature)) return NRL_E_BAD_ARG;
    if (a->flags & NRL_READOUT_MASK_BITS) {  // bit-packed: the row stride counts u32 words (0: one row for all)
        if (!a->allow_mask || (a->allow_mask & 3u) || (a->allow_row_stride != 0 && a->allow_row_stride < (a->V + 31u) / 32u)) return NRL_E_BAD_ARG;
    } else if (a->allow_mask && a->allow_row_stride != 0 && a->allow_row_stride != a->V) {
        return NRL_E_BAD_ARG;
    }
    int dev = 0, cc_major = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    if (cc_major != 10) return NRL_E_UNSUPPORTED;  // tcgen05 / tensor memory
    const uint64_t chunk = readout_chunk_rows(a->rows, a->V, a->d, a->flags);
    if (chunk >= a->rows) return readout_fwd_one(a, stream);
    if (!a->workspace || a->workspace_bytes < nrl_readout_workspace_bytes(a->rows, a->V, a->d, a->flags)) return NRL_E_WORKSPACE;
    // launches in stream order share the workspace: one launch's last kernel has read it before the next one's first writes
    for (uint64_t r0 = 0; r0 < a->rows; r0 += chunk) {
        nrl_readout_args c = *a;
        c.rows = a->rows - r0 < chunk ? a->rows - r0 : chunk;
        c.hidden = a->hidden + r0 * a->d * 2;
        if (a->tokens) c.tokens = a->tokens + r0 * 4;
        if (a->logp) c.logp = a->logp + r0 * 4;
        if (a->entropy) c.entropy = a->entropy + r0 * 4;
        if (a->rowstats) c.rowstats = a->rowstats + r0 * 16;
        if (a->status) c.status = a->status + r0;
        if (a->logits_out) c.logits_out = a->logits_out + r0 * a->V * 2;
        if (a->allow_mask) c.allow_mask = a->allow_mask + r0 * a->allow_row_stride * ((a->flags & NRL_READOUT_MASK_BITS) ? 4u : 1u);
        if (a->uniforms) c.uniforms = a->uniforms + r0 * 4;
        const int rc = readout_fwd_one(&c, stream);
        if (rc) return rc;
    }
    return NRL_OK;
}

// One launch of the readout kernel (and the kernels that finish or sample its rows) over arguments already checked.
static int readout_fwd_one(const nrl_readout_args* a, nrl_stream stream) {
    cudaError_t e = cudaSuccess;
    const bool sample = (a->flags & NRL_READOUT_SAMPLE) != 0;
    ReadoutParams p;
    memset(&p, 0, sizeof p);
    p.rows = a->rows;
    p.V = a->V;
    p.d = a->d;
    p.tiles = (a->V + kRoBN - 1) / kRoBN;
    // CTA pairs where they measured faster (B200, d = 4096, V = 128 256: 1.50 / 1.44 PFLOP/s against 1.22 / 1.27 at 8192 /
    // 18 944 rows). Beyond a few waves one CTA per block is the faster and the safer choice (1.34 against 1.15 at 65 536
    // rows): the W tiles are shared through L2 by the CTAs that walk a column range in step, a wave of 74 pairs does not
    // divide into equal groups, and groups that straddle waves fall out of step (ncu: 200 GB of DRAM reads instead of 16).
    const bool pairs = !(a->flags & NRL_READOUT_ONE_CTA) && a->rows > (uint64_t)kRoBM && a->rows <= 24576;
    p.nsplit = readout_nsplit(a->rows, a->V, a->d, pairs);
    const uint64_t unit_rows = pairs ? 2 * kRoBM : kRoBM;
    const uint64_t rb = (a->rows + unit_rows - 1) / unit_rows;  // row blocks: CTAs or CTA pairs
    if (rb * p.nsplit * 2 > 0x7fffffffull) return NRL_E_UNSUPPORTED;
    p.row_blocks = (uint32_t)rb;
    // a group (its row blocks x every column range) must not outgrow a wave, or waves would mix two groups' hidden states
    p.group_blocks = (pairs ? 74u : 148u) / p.nsplit;
    if (p.group_blocks < 1) p.group_blocks = 1;
    if (p.group_blocks > p.row_blocks) p.group_blocks = p.row_blocks;
    p.w_is_vd = (a->flags & NRL_READOUT_W_VD) ? 1u : 0u;
    p.round_bf16 = (a->flags & NRL_READOUT_ROUND_BF16) ? 1u : 0u;
    p.greedy = (a->flags & NRL_READOUT_GREEDY) ? 1u : 0u;
    p.tau = a->temperature == 0.f ? 1.f : a->temperature;
    p.tokens = (sample || p.greedy) ? nullptr : (const int32_t*)a->tokens;
    if (!a->workspace || a->workspace_bytes < readout_workspace_one(a->rows, a->V, a->d, a->flags)) return NRL_E_WORKSPACE;
    p.parts = (float*)a->workspace;
    p.allow = (const uint8_t*)a->allow_mask;
    p.allow_stride = a->allow_row_stride;
    p.allow_bits = (a->flags & NRL_READOUT_MASK_BITS) ? 1u : 0u;
    p.slog = sample ? (float2*)(a->workspace + readout_parts_bytes(a->rows, a->V, a->d)) : nullptr;
    const bool extra = sample || a->allow_mask != 0;
    p.logits_out = (uint16_t*)a->logits_out;
    CUtensorMap mx, mw;
    int rc = encode_bf16_2d(&mx, a->hidden, a->d, a->rows, kRoBK, kRoBM);
    if (rc) return rc;
    // W tiles: [V, d] as boxes of 64 k × 256 rows of W (128 for a pair: each CTA loads half a tile); [d, V] as boxes of 64 columns × 64 k
    rc = p.w_is_vd ? encode_bf16_2d(&mw, a->weights, a->d, a->V, kRoBK, pairs ? kRoBN / 2 : kRoBN) : encode_bf16_2d(&mw, a->weights, a->V, a->d, 64, kRoBK);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
#define NRL_RO_LAUNCH(KERNEL, SMEM)                                                                                  \
    do {                                                                                                            \
        e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM));                  \
        if (e != cudaSuccess) return (int)e;                                                                        \
        KERNEL<<<grid, kRoThreads, (SMEM), st>>>(mx, mw, p);                                                         \
    } while (0)
    if (pairs) {
        const uint64_t groups = (rb + p.group_blocks - 1) / p.group_blocks;
        const unsigned grid = (unsigned)(groups * p.group_blocks * p.nsplit * 2);  // one cluster of two CTAs per work item
        if (p.round_bf16) { if (extra) NRL_RO_LAUNCH((readout_fwd_pair_kernel<true, true>), kRoSmemBytes2); else NRL_RO_LAUNCH((readout_fwd_pair_kernel<true, false>), kRoSmemBytes2); }
        else              { if (extra) NRL_RO_LAUNCH((readout_fwd_pair_kernel<false, true>), kRoSmemBytes2); else NRL_RO_LAUNCH((readout_fwd_pair_kernel<false, false>), kRoSmemBytes2); }
    } else {
        const unsigned grid = (unsigned)(rb * p.nsplit);
        if (p.round_bf16) { if (extra) NRL_RO_LAUNCH((readout_fwd_kernel<true, true>), kRoSmemBytes); else NRL_RO_LAUNCH((readout_fwd_kernel<true, false>), kRoSmemBytes); }
        else              { if (extra) NRL_RO_LAUNCH((readout_fwd_kernel<false, true>), kRoSmemBytes); else NRL_RO_LAUNCH((readout_fwd_kernel<false, false>), kRoSmemBytes); }
    }
#undef NRL_RO_LAUNCH
    rc = after_launch();
    if (rc) return rc;
    if (sample) {
        const uint64_t nslabs = (uint64_t)p.tiles * (kRoBN / kRoLogCols);
        uint64_t off = readout_parts_bytes(a->rows, a->V, a->d) + ((a->rows * nslabs * sizeof(float2) + 255) & ~255ull);
        ReadoutPick* picks = (ReadoutPick*)(a->workspace + off);
        off += (a->rows * sizeof(ReadoutPick) + 255) & ~255ull;
        uint32_t* bucket_start = (uint32_t*)(a->workspace + off);
        off += ((nslabs + 1) * sizeof(uint32_t) + 255) & ~255ull;
        uint32_t* order = (uint32_t*)(a->workspace + off);
        if ((a->rows + 7) / 8 > 0x7fffffffull || a->rows > 0xffffffffull) return NRL_E_UNSUPPORTED;
        if (nslabs > (uint64_t)kRoMaxSlabs) return NRL_E_UNSUPPORTED;  // V beyond 524 288 with sampling
        readout_pick_kernel<<<(unsigned)((a->rows + 7) / 8), 256, 0, st>>>(p, (const float*)a->uniforms, picks, (int32_t*)a->tokens, (float*)a->logp, (float*)a->entropy,
                                                                           (float*)a->rowstats, (uint8_t*)a->status);
        rc = after_launch();
        if (rc) return rc;
        readout_bucket_kernel<<<1, 1024, 0, st>>>(a->rows, (uint32_t)nslabs, picks, bucket_start, order);
        rc = after_launch();
        if (rc) return rc;
        readout_draw_kernel<<<dim3(kRoDrawParts, (unsigned)nslabs), 256, 0, st>>>(p, picks, bucket_start, order, (int32_t*)a->tokens, (float*)a->logp, (const uint16_t*)a->hidden, (const uint16_t*)a->weights);
        return after_launch();
    }
    readout_finish_kernel<<<(unsigned)((a->rows + 127) / 128), 128, 0, st>>>(a->rows, p.nsplit, p.parts, (int32_t*)a->tokens, (float*)a->logp, (float*)a->entropy, (float*)a->rowstats, (uint8_t*)a->status, p.greedy);
    return after_launch();
}
