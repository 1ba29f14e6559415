/* nrl — the token-level reinforcement-learning ops of noetic-tensor's `nn::rl`, fused for
 * NVIDIA B200 (sm_100a), behind a C ABI.
 *
 * This header is what the noetic-tensor crate's hand-written FFI layer would declare beside its
 * driver-API declarations (src/tensor/cuda/ffi.rs:30-63). The conventions are that file's:
 *   - device pointers are `CUdeviceptr` values (uint64_t, src/tensor/cuda/ffi.rs:12), streams are
 *     `CUstream` (void*, src/tensor/cuda/ffi.rs:14); argument blocks are plain `#[repr(C)]` structs
 *     passed by pointer, with their size in the first field (the crate asserts its kernel
 *     parameter structs' sizes the same way, src/tensor/cuda/backend.rs:1038-1043);
 *   - every function returns an int: 0 on success, a positive value is a CUDA error code passed
 *     through (the crate wraps results with `cu(r, what)`, src/tensor/cuda/mod.rs:140-153), a
 *     negative value is one of NRL_E_* below; nothing throws, aborts or traps;
 *   - the library allocates no device memory and frees none: inputs, outputs and scratch are the
 *     caller's buffers (the crate allocates outputs from its stream-ordered pool,
 *     src/tensor/cuda/backend.rs:245-264);
 *   - work is enqueued on the caller's stream and the call returns without synchronising; the
 *     device is the one whose context is current on the calling thread (the crate makes its
 *     primary context current on entry, src/tensor/cuda/backend.rs:148-159);
 *   - tensors are contiguous and row-major: logits `[rows, V]` with rows = S·B·T, as F32 or as
 *     BF16 bit patterns (src/tensor/half.rs:16-27); tokens are I32 on the device (the crate
 *     uploads gather indices as I32, src/tensor/gpu/mod.rs:355-357); masks are one byte per element
 *     (src/tensor/gpu/mod.rs:39-40); every floating-point output is F32
 *     (src/tensor/gpu/mod.rs:335-342).
 *
 * Everything is computed in f32 with f64 only in per-row finalisation; no atomics in any
 * reduction (one shared-memory ticket counter hands out work, which does not touch results) and a
 * fixed reduction order, so results are bitwise identical from run to run on the same device.
 */
#ifndef NRL_H
#define NRL_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t nrl_devptr; /* CUdeviceptr */
typedef void* nrl_stream;    /* CUstream */

/* storage dtypes of logits */
enum { NRL_F32 = 0, NRL_BF16 = 1 };

/* error codes (negative); positive return values are cudaError_t / CUresult numbers */
enum {
    NRL_OK = 0,
    NRL_E_BAD_ARG = -1,     /* null pointer, zero size, struct_size mismatch, misaligned pointer */
    NRL_E_UNSUPPORTED = -2, /* dtype / option this build has no kernel for */
    NRL_E_WORKSPACE = -3,   /* scratch buffer missing or too small */
    NRL_E_ROW_STATUS = -4,  /* reported by nrl_check_status: a row had no allowed token or a NaN */
    NRL_E_NO_DEVICE = -5,   /* no CUDA device / no current context */
    NRL_E_NOT_FINITE = -6   /* reported by nrl_check_scored_finite: a scored log-probability is -inf, +inf or NaN */
};

/* ---------------------------------------------------------------------------------------------
 * Library identity.
 * nrl_key replaces `CudaBackend::key` (src/tensor/cuda/backend.rs:962-966): a provenance string
 * naming what results depend on, ending in the first 16 hex digits of the SHA-256 of the kernel
 * sources. */
int nrl_version(void);
const char* nrl_key(void);
const char* nrl_error_string(int code);
/* Kernels launched by this library in this process so far (the crate's `launches()`,
 * src/tensor/cuda/backend.rs:1032-1036). */
uint64_t nrl_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * Row forward: one streaming pass over each vocabulary row.
 *
 * Replaces, for a `Device::Cuda` tensor, the op sequences of
 *   tempered_logits      src/nn/rl.rs:475-486   (z = logits / temperature + additive mask)
 *   sample_categorical   src/nn/rl.rs:510-529   (here: inverse CDF against one uniform per row,
 *                                                or the first maximum when NRL_FWD_GREEDY)
 *   token_log_probs      src/nn/rl.rs:134-141   (log_softmax(z)[token], src/tensor/activation.rs:30-35)
 *   categorical_kl /     src/nn/rl.rs:327-351   (per-row exact KL(softmax z ‖ softmax z_ref), both
 *   reference_kl                                 sides tempered and masked alike)
 *   categorical_entropy  src/nn/rl.rs:405-414   (per-row entropy)
 * and saves the per-row statistics the backward needs in place of log_softmax's saved output
 * (src/tensor/autodiff.rs:110-119).
 *
 * Sampling: with z the tempered, masked logits of a row in f32, m = max z, e_v = exp(z_v − m),
 * Z = Σ e_v, the token is min{k : Σ_{v≤k} e_v > u·Z} for the row's uniform u in [0, 1).
 * A row with no allowed token or with a NaN gets token −1, NaN outputs and a non-zero status byte
 * (bit 0: no allowed token; bit 1: NaN), where the reference panics (src/nn/rl.rs:516-519).
 *
 * KL where the two sides exclude different tokens (src/nn/rl.rs:322-325 asks for the same
 * vocabulary mask on both sides; the allow-mask here always applies to both): a token whose
 * policy logit is −inf contributes 0 whatever the reference holds, as in the reference
 * (`mask_fill(zero_p, 0)`). A token the reference excludes (z_ref = −inf) while the policy's logit
 * is finite makes the row's KL non-finite, as in the reference: +inf while π_v > 0 in f32, NaN once
 * π_v has underflowed to 0 (0·inf). The two underflow at different points: the reference's
 * `exp(logp)` at logp < −103.97 (f32 denormals), this library's flush-to-zero exponential at
 * z_v − m < −87.34; in between the reference gives +inf and this library NaN. The backward of such
 * a row is NaN in every entry (KL enters every entry of the gradient).
 */
enum {
    NRL_FWD_SAMPLE = 1u << 0,  /* draw tokens (needs `uniforms`, writes `tokens`) */
    NRL_FWD_GREEDY = 1u << 1,  /* tokens = first maximum of z (temperature 0); writes `tokens` */
    NRL_FWD_TOKENS_IN = 1u << 2, /* `tokens` is an input (token_log_probs of given tokens) */
    NRL_FWD_MASK_BITS = 1u << 3, /* `allow_mask` is bit-packed (no counterpart in the reference, whose masks are a byte or an
                                    f32 per token): u32 words, bit v of a row = bit (v mod 32) of its word v / 32, and
                                    `allow_row_stride` counts WORDS between rows (>= ceil(V / 32), or 0 for one row
                                    broadcast). The kernels read V / 8 mask bytes per row instead of V */
    NRL_FWD_ROW_PER_BLOCK = 1u << 4 /* always take the kernel that gives every row a thread block of its own, also for the
                                    many-row shapes that otherwise run the kernel in which a block owns a group of rows.
                                    The two split a row into parts differently, so results agree to rounding, not to the
                                    bit; each is reproducible run to run. For comparisons and for callers that must get
                                    the same bits whatever the number of rows in the call */
};

typedef struct nrl_row_fwd_args {
    uint32_t struct_size;      /* sizeof(nrl_row_fwd_args) */
    uint32_t flags;            /* NRL_FWD_* ; at most one of SAMPLE / GREEDY / TOKENS_IN */
    uint32_t dtype;            /* dtype of `logits` and of `ref_logits` */
    uint32_t V;                /* vocabulary size, ≥ 1 */
    uint64_t rows;             /* S·B·T */
    float temperature;         /* τ as f32; 1.0 leaves the logits as they are; must be > 0 */
    uint32_t reserved0;
    nrl_devptr logits;         /* [rows, V] */
    nrl_devptr ref_logits;     /* [rows, V] or 0: frozen reference (detached) */
    nrl_devptr allow_mask;     /* u8, non-zero = allowed; [rows, V], or [1, V] with stride 0; or 0 */
    uint64_t allow_row_stride; /* elements between rows of allow_mask: V or 0 */
    nrl_devptr add_mask;       /* f32 additive mask (−inf or −1e9 exclude), [rows, V] or [1, V]; or 0 */
    uint64_t add_row_stride;   /* V or 0 */
    nrl_devptr uniforms;       /* f32 [rows] in [0,1), for NRL_FWD_SAMPLE; else 0 */
    nrl_devptr tokens;         /* i32 [rows]: output (SAMPLE, GREEDY) or input (TOKENS_IN); or 0 */
    nrl_devptr logp;           /* out f32 [rows]: log-prob of the token under z; or 0 */
    nrl_devptr ref_logp;       /* out f32 [rows]: log-prob of the token under z_ref; or 0 */
    nrl_devptr kl;             /* out f32 [rows]: exact KL; or 0 */
    nrl_devptr entropy;        /* out f32 [rows]; or 0 */
    nrl_devptr rowstats;       /* out f32 [rows, 4] = (m, ln Z, m_ref, ln Z_ref) for nrl_row_bwd; or 0 */
    nrl_devptr status;         /* out u8 [rows]; or 0 */
    nrl_devptr workspace;      /* scratch, nrl_row_fwd_workspace_bytes(rows, V) bytes; may be 0 if that is 0 */
    uint64_t workspace_bytes;
} nrl_row_fwd_args;

/* Scratch bytes nrl_row_fwd needs for this shape: 0 when every row gets a whole thread block,
 * non-zero when few long rows are split over several blocks each. */
uint64_t nrl_row_fwd_workspace_bytes(uint64_t rows, uint32_t V);
int nrl_row_fwd(const nrl_row_fwd_args* args, nrl_stream stream);

/* The same forward for callers that have no device allocator to take scratch memory from.
 * (No counterpart in the reference: there every op allocates its outputs from the crate's own
 * stream-ordered pool.) Some hosts of this library cannot call cudaMalloc at the point where they
 * sample: an inference server that has handed all device memory to its own arena at start-up, a
 * decode loop running under a no-allocation rule, or a plugin that is given buffers but no
 * allocator. For them this entry point needs only the inputs and outputs in `args`: when few long
 * rows are split over several thread blocks, the per-block partial results go to a fixed
 * NRL_STATIC_SCRATCH_BYTES array that lives inside the library's device image (each GPU that loads
 * the library holds that much memory until the process exits). `args->workspace` and
 * `args->workspace_bytes` are ignored. It never calls cudaMalloc, cudaFree or any allocating
 * routine.
 *   - A shape whose scratch need (nrl_row_fwd_workspace_bytes) exceeds NRL_STATIC_SCRATCH_BYTES is
 *     refused with NRL_E_WORKSPACE before anything is launched.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current). Make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one array. Nothing in it needs to start at zero (every slot
 *     that is read is written earlier in the same call), and it keeps the last call's contents.
 *     Two calls whose kernels may overlap on the GPU (different streams, no ordering) race on
 *     it: order them, or use nrl_row_fwd with separate workspaces. */
#define NRL_STATIC_SCRATCH_BYTES (64u * 1024u)
int nrl_row_fwd_static(const nrl_row_fwd_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Row backward: d(logits) in one streaming pass.
 *
 * Replaces the tape's backward of the same functions (gather → scatter_add into a dense
 * one-hot, src/tensor/float.rs:1004-1011, 1049-1054; log_softmax backward g − exp(y)·Σg,
 * src/tensor/activation.rs:36-41; the exp / mul / mask_fill / sum_dim nodes of categorical_kl and
 * categorical_entropy). With π = softmax(z), ρ = softmax(z_ref) and the per-row upstream
 * gradients g_lp, g_kl, g_ent of the row's log-prob, KL and entropy:
 *   dz_j = g_lp·(1[j = token] − π_j) + g_kl·π_j·(log π_j − log ρ_j − KL) − g_ent·π_j·(log π_j + H)
 * and d(logits) = dz / temperature. Entries with π_j = 0 get exactly 0; rows whose three
 * upstream gradients are all zero (unscored positions) are written as exact zeros without
 * reading the logits.
 */
typedef struct nrl_row_bwd_args {
    uint32_t struct_size;
    uint32_t dtype;
    uint32_t V;
    float temperature;
    uint64_t rows;
    nrl_devptr logits;
    nrl_devptr ref_logits; /* or 0 (then g_kl must be 0) */
    nrl_devptr allow_mask;
    uint64_t allow_row_stride;
    nrl_devptr add_mask;
    uint64_t add_row_stride;
    nrl_devptr tokens;   /* i32 [rows], or 0 (then g_lp must be 0) */
    nrl_devptr rowstats; /* f32 [rows, 4] from nrl_row_fwd */
    nrl_devptr kl;       /* f32 [rows] from nrl_row_fwd, or 0 when g_kl is 0 */
    nrl_devptr entropy;  /* f32 [rows] from nrl_row_fwd, or 0 when g_ent is 0 */
    nrl_devptr g_logp;   /* f32 [rows] or 0 */
    nrl_devptr g_kl;     /* f32 [rows] or 0 */
    nrl_devptr g_ent;    /* f32 [rows] or 0 */
    nrl_devptr d_logits; /* out f32 [rows, V] */
    uint32_t accumulate; /* 1: add into d_logits instead of overwriting it (the tape's `new + old`,
                            src/tensor/autodiff.rs:198-201, without a separate pass) */
    uint32_t mask_bits;  /* 1: allow_mask is bit-packed as with NRL_FWD_MASK_BITS (allow_row_stride in words) */
    nrl_devptr g_uniform;    /* f32 [rows] or 0: upstream gradient of −mean_v log π_v (the label-smoothing
                                term of cross_entropy_with, src/nn/loss.rs:70-72); adds g·(π_j − 1/V).
                                Not with masks or a temperature (NRL_E_UNSUPPORTED) */
    nrl_devptr d_ref_logits; /* out f32 [rows, V] or 0: gradient w.r.t. ref_logits of the KL term,
                                g_kl·(ρ_j − π_j) (kl_div's prediction side, src/nn/loss.rs:175-183).
                                With it, d_logits may be 0 (a detached teacher) */
} nrl_row_bwd_args;

int nrl_row_bwd(const nrl_row_bwd_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Token-level losses over `[S, B, T]` values, forward and the derivative with respect to logp.
 *
 *   NRL_LOSS_PG   policy_gradient_loss  src/nn/rl.rs:228-235   l = −w·logp
 *   NRL_LOSS_PPO  clipped_policy_loss   src/nn/rl.rs:265-287   with Clip (src/nn/rl.rs:160-198),
 *                 log_ratio (:239-246), select_max (:124-129), the dual clip (:276-285)
 *   NRL_LOSS_K1/K2/K3  kl_estimate      src/nn/rl.rs:380-400   δ = other − logp, optional clamp
 * Unscored positions (mask 0) give exactly 0 and exactly zero derivative, by a select
 * (zero_masked, src/nn/rl.rs:99-102). The derivative follows the tape's rules: clamps and
 * selects pass no gradient where they are active (src/tensor/float.rs:578-594, 984-1000).
 */
enum { NRL_LOSS_PG = 0, NRL_LOSS_PPO = 1, NRL_LOSS_K1 = 2, NRL_LOSS_K2 = 3, NRL_LOSS_K3 = 4 };

typedef struct nrl_token_loss_args {
    uint32_t struct_size;
    uint32_t kind;        /* NRL_LOSS_* */
    uint64_t S, B, T;
    nrl_devptr logp;      /* f32 [S,B,T] */
    nrl_devptr other;     /* PPO: old log-probs; K1..K3: reference log-probs; PG: 0 */
    nrl_devptr weights;   /* PG: weights; PPO: advantages; [S,B,T] or [S,B]; K*: 0 */
    uint32_t weights_per_sequence; /* 1: weights are [S,B] */
    uint32_t has_dual;
    nrl_devptr mask;      /* f32 [S,B,T] of 0/1, or 0 (every position scored) */
    double clip_low, clip_high; /* PPO: the ratio is clipped to [(f32)(1 − low), (f32)(1 + high)] */
    double dual;          /* PPO: dual-clip constant c > 1, used when has_dual */
    double clamp;         /* PPO: log-ratio clamp; K*: δ clamp; used when has_clamp */
    uint32_t has_clamp;
    uint32_t accumulate;  /* 1: add into dloss_dlogp instead of overwriting it (a logp tensor that feeds two losses) */
    nrl_devptr loss;      /* out f32 [S,B,T], 0 at unscored positions; or 0 */
    nrl_devptr upstream;  /* f32 [S,B,T] gradient of the per-token loss (from nrl_reduce_tokens_bwd), or 0 for ones */
    nrl_devptr dloss_dlogp; /* out f32 [S,B,T] = upstream · d loss / d logp; or 0 */
} nrl_token_loss_args;

int nrl_token_loss(const nrl_token_loss_args* args, nrl_stream stream);

/* clip_fraction (src/nn/rl.rs:293-317): per seed, the fraction of scored tokens whose gradient a
 * bound of clipped_policy_loss removes. Same inputs as NRL_LOSS_PPO; out f32 [S]. */
int nrl_clip_fraction(const nrl_token_loss_args* args, nrl_devptr out_fraction, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * TokenReduction (src/nn/rl.rs:36-55, reduce_tokens :69-86, per_sequence :88-92).
 * `per` must already be zero at unscored positions (the losses above and nrl_mask_rows do that).
 * Forward: out is [S] (SUM, TOKEN_MEAN, SEQUENCE_MEAN), [S,B] (PER_SEQUENCE) or a copy (NONE).
 * Backward: d_per[s,b,t] from the upstream gradient of the reduced value, exactly 0 at unscored
 * positions. Sums run in a fixed tree order.
 */
enum { NRL_REDUCE_NONE = 0, NRL_REDUCE_SUM = 1, NRL_REDUCE_TOKEN_MEAN = 2, NRL_REDUCE_PER_SEQUENCE = 3, NRL_REDUCE_SEQUENCE_MEAN = 4 };

int nrl_reduce_tokens(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, nrl_devptr per, nrl_devptr mask, nrl_devptr out, nrl_stream stream);
int nrl_reduce_tokens_bwd(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, nrl_devptr mask, nrl_devptr g_out, nrl_devptr d_per, nrl_stream stream);

/* The same reductions when the sequences of one job live on several GPUs (one process per device,
 * src/tensor/cuda/backend.rs:106-138; the seed axis is partitioned, then B). The reduction has two
 * fixed steps: one warp sums a sequence to the pair (sum of per, sum of mask); a seed's pairs are
 * folded in sequence order in f64 (reduce_tokens and per_sequence, src/nn/rl.rs:69-92).
 * nrl_reduce_tokens runs both; a sharded caller runs step 1 on the sequences it holds
 * (nrl_reduce_tokens_partial: `per`, `mask` f32 [n_seq, T] -> `pairs` f32 [n_seq, 2]), gathers the
 * pairs of all S*B sequences in sequence order (a few bytes per sequence: the one collective of
 * the path) and runs step 2 (nrl_reduce_tokens_fold: `pairs` f32 [S*B, 2] -> out [S] or [S, B]).
 * The result has the bits of nrl_reduce_tokens on one GPU, for any number of GPUs.
 * nrl_reduce_tokens_bwd_pairs is the backward for such a caller: it holds sequences
 * [seq_begin, seq_begin + n_seq) of the S*B (flat index s*B + b); `pairs` are the gathered pairs of
 * all sequences (their counts give the divisors), `mask` and `d_per` cover the local sequences
 * [n_seq, T], `g_out` is the gradient of the whole reduced value ([S] or [S, B]; for
 * NRL_REDUCE_NONE the local [n_seq, T], and `pairs` may be 0). */
int nrl_reduce_tokens_partial(uint64_t n_seq, uint64_t T, nrl_devptr per, nrl_devptr mask, nrl_devptr pairs, nrl_stream stream);
int nrl_reduce_tokens_fold(uint32_t reduction, uint64_t S, uint64_t B, nrl_devptr pairs, nrl_devptr out, nrl_stream stream);
int nrl_reduce_tokens_bwd_pairs(uint32_t reduction, uint64_t S, uint64_t B, uint64_t T, uint64_t seq_begin, uint64_t n_seq, nrl_devptr pairs, nrl_devptr mask,
                                nrl_devptr g_out, nrl_devptr d_per, nrl_stream stream);

/* A whole token-level objective in one launch (no single counterpart in the reference, which
 * composes it from the functions above): the token loss `policy` (any NRL_LOSS_* kind) of the
 * log-probs, and the per-token exact KL and entropy that nrl_row_fwd left (either may be 0), all
 * three under the same scoring mask and the same per-seed TokenReduction (SUM, TOKEN_MEAN or
 * SEQUENCE_MEAN; the others: NRL_E_UNSUPPORTED), and at once the per-token upstream gradients
 * nrl_row_bwd takes. It stands for nrl_token_loss + three nrl_reduce_tokens + three
 * nrl_reduce_tokens_bwd + the backward nrl_token_loss — eight launches — and gives their bits:
 *   out_policy[s] = reduce(token_loss(policy))        g_logp[i] = d_per_policy[i] · d loss_i / d logp_i
 *   out_kl[s]     = reduce(zero_masked(kl))           g_kl[i]   = d_per_kl[i]
 *   out_entropy[s]= reduce(zero_masked(entropy))      g_ent[i]  = d_per_entropy[i]
 * where d_per_x is what nrl_reduce_tokens_bwd gives for the upstream gradient up_x [S] of the reduced
 * value (0 = ones). A caller forms its objective from the three reduced values (for example
 * policy + 0.04·kl − 0.01·entropy) and passes the matching upstream gradients (1, 0.04, −0.01). */
typedef struct nrl_token_objective_args {
    uint32_t struct_size;
    uint32_t reduction;           /* NRL_REDUCE_SUM, NRL_REDUCE_TOKEN_MEAN or NRL_REDUCE_SEQUENCE_MEAN */
    nrl_token_loss_args policy;   /* kind, S, B, T, logp, other, weights, mask, clip constants; its loss / upstream / dloss_dlogp / accumulate fields are ignored */
    nrl_devptr kl;                /* f32 [S,B,T] per-token exact KL, or 0 */
    nrl_devptr entropy;           /* f32 [S,B,T] per-token entropy, or 0 */
    nrl_devptr up_policy, up_kl, up_entropy;    /* f32 [S] each, or 0 for ones */
    nrl_devptr out_policy, out_kl, out_entropy; /* out f32 [S] each, or 0 */
    nrl_devptr g_logp, g_kl, g_ent;             /* out f32 [S,B,T] each, or 0 */
} nrl_token_objective_args;

int nrl_token_objective(const nrl_token_objective_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * The cross-entropy family of nn::loss over the same row kernels (src/nn/loss.rs:10-79):
 *   nll                    :10-16   −log_softmax(logits)[target]           = −logp of nrl_row_fwd(TOKENS_IN)
 *   cross_entropy          :19-22   per-seed mean of nll
 *   masked_cross_entropy   :27-34   Σ(nll·mask) / max(Σmask, 1)
 *   cross_entropy_with     :48-79   + ignore_index (host: target → class 0, keep → 0) and label
 *                                   smoothing ε: (1 − ε)·nll + ε·(−mean_v log π_v)
 * replacing log_softmax → dense one-hot [S, N, V] product → lane sum. The mask enters as a product
 * (as the reference's `nll * mask`), so a non-finite loss at an unscored position gives NaN there too.
 *
 * nrl_row_sum: out[r] = Σ_v logits[r, v] in f32, fixed order (needed only for ε > 0:
 * −mean_v log π_v = m + ln Z − Σ_v z_v / V).
 * nrl_ce_tokens: the O(rows) part. Forward: loss[i] = ((1 − ε)·(−logp[i]) + ε·u[i])·keep[i].
 * Backward (when `upstream` is given): g_logp[i] = −(1 − ε)·keep[i]·upstream[i] and
 * g_uniform[i] = ε·keep[i]·upstream[i], the per-row gradients nrl_row_bwd takes.
 * Per-seed means are nrl_reduce_tokens(NRL_REDUCE_TOKEN_MEAN, S, 1, N, loss, keep, out). */
int nrl_row_sum(uint32_t dtype, uint64_t rows, uint32_t V, nrl_devptr logits, nrl_devptr out, nrl_stream stream);

typedef struct nrl_ce_args {
    uint32_t struct_size;
    uint32_t V;
    uint64_t n;            /* S·B·T positions */
    double smoothing;      /* ε in [0, 1] */
    nrl_devptr logp;       /* f32 [n]: log-prob of the target (nrl_row_fwd, NRL_FWD_TOKENS_IN) */
    nrl_devptr rowstats;   /* f32 [n, 4] of the same call; read when ε > 0 */
    nrl_devptr logit_sum;  /* f32 [n] from nrl_row_sum; read when ε > 0 */
    nrl_devptr keep;       /* f32 [n] mask × not-ignored, or 0 for all ones */
    nrl_devptr loss;       /* out f32 [n], or 0 */
    nrl_devptr upstream;   /* f32 [n] gradient of loss (from nrl_reduce_tokens_bwd), or 0 for no backward */
    nrl_devptr g_logp;     /* out f32 [n] (with upstream) */
    nrl_devptr g_uniform;  /* out f32 [n] (with upstream and ε > 0), else 0 */
} nrl_ce_args;

int nrl_ce_tokens(const nrl_ce_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * The reference's own sampler on the device (sample_categorical + gumbel, src/nn/rl.rs:490-529):
 * Gumbel-max with one ChaCha20 `next_u64` per logit in row-major order,
 *   k = next_u64() >> 11;  u = (k + 1/2) / 2^53;  g = (f32)(-ln(-ln u));  token = first max of z + g,
 * z = logits / temperature + mask in f32. The stream is rand_chacha 0.3's ChaCha20Rng of `seed`
 * (20 rounds, 64-bit block counter, zero stream id; u64 = two consecutive 32-bit words, low
 * first), entered `word_offset` 32-bit words after its start, so tokens equal the reference's for
 * the same seed and position (its noise logarithms are glibc's, here CUDA's: both within 1 ulp in
 * f64 before the cast to f32). The call consumes 2 * rows * V words: a caller that keeps drawing
 * from the same generator advances its position by that much.
 * temperature = 0 (greedy, no draws) is nrl_row_fwd with NRL_FWD_GREEDY. A row with no allowed
 * token or a NaN gets token -1 and a status byte as in nrl_row_fwd (the reference panics before
 * drawing anything, src/nn/rl.rs:516-519; check the status before using the generator further). */
typedef struct nrl_gumbel_args {
    uint32_t struct_size;
    uint32_t dtype;
    uint32_t V;
    float temperature;         /* > 0 */
    uint64_t rows;
    nrl_devptr logits;         /* [rows, V] */
    nrl_devptr allow_mask;     /* u8 as in nrl_row_fwd, or 0 */
    uint64_t allow_row_stride;
    nrl_devptr add_mask;       /* f32 additive mask as in nrl_row_fwd, or 0 */
    uint64_t add_row_stride;
    uint8_t seed[32];          /* the ChaCha20 key (rng::derive's SHA-256, src/rng.rs:10-17) */
    uint64_t word_offset;      /* 32-bit words already drawn from the generator */
    nrl_devptr tokens;         /* out i32 [rows] */
    nrl_devptr status;         /* out u8 [rows], or 0 */
} nrl_gumbel_args;

int nrl_sample_gumbel(const nrl_gumbel_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Rows that live in HOST memory (no counterpart in the reference, whose tensors are uploaded
 * whole, src/tensor/gpu/mod.rs:472-481): the byte-masked forward never reads a logit the mask
 * excludes, so those need not cross PCIe.
 * nrl_host_pack runs on `threads` host threads (no CUDA call): per row it writes one liveness bit
 * per 8-element vector (a vector is live when any of its 8 mask bytes is non-zero) and, for the
 * live vectors in row order, their logits, reference logits and 8 mask bytes. The output arrays
 * are the caller's (pinned, for the copies that follow). Returns NRL_E_WORKSPACE with
 * `live_vectors` set when `capacity` is too small: upload the rows whole instead.
 * nrl_unpack_rows (one kernel) takes the device copies of those arrays and writes the live vectors
 * to their places in the full [rows, V] logits / reference buffers and the full byte mask (zeros
 * for the rest); other elements of the logits buffers keep whatever they held. The buffers are
 * then what nrl_row_fwd / nrl_row_bwd take with that mask. V must be a multiple of 8, V <= 262144. */
typedef struct nrl_pack_args {
    uint32_t struct_size;
    uint32_t dtype;
    uint32_t V;
    uint32_t threads;
    uint64_t rows;
    const void* logits;         /* host [rows, V] */
    const void* ref_logits;     /* host [rows, V] or NULL */
    const uint8_t* allow_mask;  /* host u8 [rows, V] */
    uint64_t capacity;          /* live vectors the packed arrays can hold */
    uint64_t* live_words;       /* out host u64 [rows, ceil(V / 8 / 64)]: bit j of word w = vector 64w + j is live */
    uint32_t* row_offset;       /* out host u32 [rows + 1]: live vectors before each row */
    void* packed_logits;        /* out host [capacity, 8] elements */
    void* packed_ref;           /* out host [capacity, 8] elements, or NULL */
    uint64_t* packed_mask;      /* out host [capacity]: the 8 mask bytes of each live vector */
    uint64_t live_vectors;      /* out */
} nrl_pack_args;

int nrl_host_pack(nrl_pack_args* args);

typedef struct nrl_unpack_args {
    uint32_t struct_size;
    uint32_t dtype;
    uint32_t V;
    uint32_t reserved0;
    uint64_t rows;
    nrl_devptr live_words, row_offset, packed_logits, packed_ref, packed_mask; /* device copies of nrl_host_pack's outputs */
    nrl_devptr logits;      /* out [rows, V]: live vectors written */
    nrl_devptr ref_logits;  /* out [rows, V] or 0 (with packed_ref 0) */
    nrl_devptr allow_mask;  /* out u8 [rows, V]: written in full */
} nrl_unpack_args;

int nrl_unpack_rows(const nrl_unpack_args* args, nrl_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Generic reductions along the last axis of a contiguous [rows, V] tensor, one block per row with
 * 64-bit offsets. They replace the CUDA backend's lane kernels, which put ONE THREAD on a whole
 * row (sum_last_f32, argmax_dim_f32: src/tensor/cuda/kernels.rs:625-670) and compose softmax,
 * log_softmax and logsumexp from 6 generic launches each (src/tensor/activation.rs:15-42, 71-77).
 *   NRL_LANE_SOFTMAX         out[r, :] = exp(x − max) / Σ exp(x − max)         activation.rs:15-26
 *   NRL_LANE_LOG_SOFTMAX     out[r, :] = (x − max) − log Σ exp(x − max)         activation.rs:30-42
 *   NRL_LANE_LOGSUMEXP       out[r] = m + log Σ exp(x − m), m = 0 where max is ±inf  activation.rs:71-77
 *   NRL_LANE_ARGMAX          out_index[r] (i32) = first maximum, the first NaN if the row holds one;
 *                            out (optional, f32 [rows]) = its value           kernels.rs:184-209
 *   NRL_LANE_SUM             out[r] = Σ_v x[r, v] in the reference's operand order (eight partial
 *                            sums, (p0+p4)+(p1+p5)+(p2+p6)+(p3+p7), then the tail): bit-equal to
 *                            Cpu(Reference) and to sum_last_f32                kernels.rs:122-148
 *   NRL_LANE_SOFTMAX_BWD     out = y · (g − Σ g·y)      x = the saved output y (f32), g f32 [rows, V]
 *   NRL_LANE_LOG_SOFTMAX_BWD out = g − exp(y) · Σ g     x = the saved output y (f32), g f32 [rows, V]
 *   NRL_LANE_LOGSUMEXP_BWD   out = g[r] · exp(x − lse[r])   x = the input, lse = the saved output, g f32 [rows]
 * x is F32 or BF16 for the forward ops and for NRL_LANE_LOGSUMEXP_BWD, F32 for the other two
 * backward ops. Outputs are F32. A row of −inf alone, or one holding NaN, gives NaN from softmax and
 * log_softmax as in the reference. `out` must not alias an input. Rows take 16-byte loads when V
 * is a multiple of 8 and x, g, out are 16-byte aligned; other shapes run an element-wise loop.
 * softmax / log_softmax of such rows longer than 42 KB (and up to 896 KB) run on thread-block
 * clusters that hold a row in shared memory and read it from HBM once; the CTAs of a cluster wait
 * for each other's partial sums at most two seconds, after which the CTA writes NaN rows (an internal
 * error: it cannot happen unless a CTA of the cluster has faulted). Results do not depend on timing. */
enum {
    NRL_LANE_SOFTMAX = 0, NRL_LANE_LOG_SOFTMAX = 1, NRL_LANE_LOGSUMEXP = 2, NRL_LANE_ARGMAX = 3, NRL_LANE_SUM = 4,
    NRL_LANE_SOFTMAX_BWD = 5, NRL_LANE_LOG_SOFTMAX_BWD = 6, NRL_LANE_LOGSUMEXP_BWD = 7
};

typedef struct nrl_lane_args {
    uint32_t struct_size;
    uint32_t op;
    uint32_t dtype;        /* of x */
    uint32_t V;
    uint64_t rows;
    nrl_devptr x;          /* [rows, V] */
    nrl_devptr g;          /* backward ops: upstream gradient */
    nrl_devptr lse;        /* NRL_LANE_LOGSUMEXP_BWD: f32 [rows] */
    nrl_devptr out;        /* f32 [rows, V] or [rows]; optional for NRL_LANE_ARGMAX */
    nrl_devptr out_index;  /* NRL_LANE_ARGMAX: i32 [rows] */
} nrl_lane_args;

int nrl_lane_op(const nrl_lane_args* args, nrl_stream stream);

/* Bit-packed vocabulary masks (no counterpart in the reference, whose masks are one byte or one
 * f32 per token, src/tensor/gpu/mod.rs:39-40): `bits` holds u32 words, bit v of a row being bit
 * (v mod 32) of its word v / 32, rows `bits_row_stride_words` words apart (0 = one row broadcast
 * to all). nrl_expand_bitmask writes the U8 allow-mask [rows, V] (0 / 1) that nrl_row_fwd and
 * nrl_row_bwd take: a host caller uploads V / 8 bytes per row instead of V. */
/* The other direction, on `threads` host threads (no CUDA call): a host byte mask u8 [rows, V] to
 * bit-packed words u32 [rows, ceil(V / 32)] in the layout above, for callers whose rows live in
 * host memory: the mask then crosses the host link as V / 8 bytes per row. */
int nrl_host_pack_bits(uint64_t rows, uint32_t V, const uint8_t* allow_mask, uint32_t* bits, uint32_t threads);

int nrl_expand_bitmask(uint64_t rows, uint32_t V, nrl_devptr bits, uint64_t bits_row_stride_words, nrl_devptr allow_mask, nrl_stream stream);

/* zero_masked (src/nn/rl.rs:99-102) of per-row values: out[i] = mask[i] == 0 ? 0 : x[i]. */
int nrl_mask_rows(uint64_t n, nrl_devptr x, nrl_devptr mask, nrl_devptr out, nrl_stream stream);

/* group_advantages_tensor (src/nn/rl.rs:436-469) without the host round trip: rewards f32
 * [groups, n] on the device -> advantages f32 [groups, n], each reward minus its group's mean and,
 * with norm_std, divided by the group's standard deviation (sample when `unbiased`, which needs
 * n >= 2) plus eps. Computed in f64 in the host function's operand order and rounded to f32 once,
 * so the values are the reference's bit for bit; a group whose rewards are all equal gives exact
 * zeros. NRL_E_BAD_ARG for eps < 0 or unbiased with n < 2 (the reference's assertions). */
int nrl_group_advantages(uint64_t groups, uint32_t n, uint32_t norm_std, double eps, uint32_t unbiased, nrl_devptr rewards, nrl_devptr out, nrl_stream stream);

/* Reads `status` (u8 [rows], device) back and returns NRL_E_ROW_STATUS with the first bad row in
 * *first_bad_row if any byte is non-zero. Synchronises the stream: this is the host read the
 * reference's sampler does (src/nn/rl.rs:516-519). */
int nrl_check_status(nrl_devptr status, uint64_t rows, nrl_stream stream, uint64_t* first_bad_row, uint32_t* bits);

/* ---------------------------------------------------------------------------------------------
 * Readout-fused row statistics: the step before the path taken into it. The reference computes
 * logits = hidden · W with `Decoder::head` (src/nn/decoder.rs:270-279; `Linear` holds W as
 * [in, out] = [d, V], src/nn/linear.rs:1-3, 51-58), on CUDA through `hgemm_bf16_f32acc`
 * (src/tensor/cuda/half_gemm.rs:32-168: operands rounded to bf16, f32 accumulators,
 * mma.sync.m16n8k16), writes the [rows, V] logits and then reads them back in token_log_probs /
 * categorical_entropy (src/nn/rl.rs:134-141, 405-414). nrl_readout_fwd does the product on the
 * B200 tensor cores (tcgen05.mma, bf16 operands, f32 accumulators in tensor memory, TMA-fed) and
 * folds each finished 128 × 256 tile of logits into the rows' maximum, log-sum-exp and entropy
 * sums straight from tensor memory, so the logits are never written or re-read:
 *   rowstats[r] = (m, ln Z, 0, 0), entropy[r] = ln Z − Σ e_v (z_v − m) / Z,
 *   logp[r] = z_token − m − ln Z for the given token (NRL_FWD_TOKENS_IN semantics) or, with
 *   NRL_READOUT_SAMPLE, for the token drawn by inverse CDF against the row's uniform; an optional
 *   byte allow-mask excludes tokens as in nrl_row_fwd (tempered_logits' −inf mask),
 * with z = the f32 accumulators (the reference's logits are f32 too), or, with
 * NRL_READOUT_ROUND_BF16, z rounded to bf16 first — what a bf16 logits tensor handed to
 * nrl_row_fwd would hold. `hidden` is bf16 [rows, d], `weights` bf16 [d, V] (the reference's
 * layout) or, with NRL_READOUT_W_VD, [V, d]; d and V multiples of 8, both 16-byte aligned.
 * `logits_out` (optional, bf16 [rows, V]) receives the rounded logits, for comparisons.
 * Needs compute capability 10.x (NRL_E_UNSUPPORTED otherwise) and
 * nrl_readout_workspace_bytes(rows, V, d, flags) bytes of scratch. status[r]: bit 0 no finite logit, bit 1
 * a NaN, bit 2 the kernel gave up a bounded wait (an internal error: outputs of that row are NaN).
 * Results are bitwise reproducible run to run. */
enum {
    NRL_READOUT_W_VD = 1u << 0,
    NRL_READOUT_ROUND_BF16 = 1u << 1,
    NRL_READOUT_SAMPLE = 1u << 3,  /* draw the tokens (inverse CDF against `uniforms`, as NRL_FWD_SAMPLE) instead of taking them:
                                     `tokens` is then an output and `logp` the drawn tokens' log-probs. The pass logs each
                                     row's mass per 64 columns; a second small kernel finds the 64 columns holding u·Z and
                                     computes those 64 logits again (f32) to walk to the token */
    NRL_READOUT_GREEDY = 1u << 4,  /* the token is the row's first maximum (sample_categorical at temperature 0, src/nn/rl.rs:510-529): `tokens` is an
                                     output, `logp` its log-prob; the allow-mask applies; not together with NRL_READOUT_SAMPLE */
    NRL_READOUT_MASK_BITS = 1u << 5,  /* `allow_mask` holds one bit per token (u32 words, bit v mod 32 of word v / 32, as NRL_FWD_MASK_BITS);
                                        `allow_row_stride` then counts words per row (≥ ceil(V / 32), or 0 for one row shared by all) */
    NRL_READOUT_ONE_CTA = 1u << 2 /* one CTA per 128-row block (tcgen05 cta_group::1) instead of CTA pairs on 256-row blocks
                                    (cta_group::2, the default for more than 128 rows), and one launch however many rows: the same bits up to
                                    24 576 rows; beyond, the count of column ranges, and with it the last bits of the sums, may differ */
};

typedef struct nrl_readout_args {
    uint32_t struct_size;
    uint32_t flags;          /* NRL_READOUT_* */
    uint32_t V;              /* vocabulary size, a multiple of 8 */
    uint32_t d;              /* model width, a multiple of 8 */
    uint64_t rows;           /* S·B·T */
    nrl_devptr hidden;       /* bf16 [rows, d] */
    nrl_devptr weights;      /* bf16 [d, V], or [V, d] with NRL_READOUT_W_VD */
    nrl_devptr tokens;       /* i32 [rows] given tokens, or 0 */
    nrl_devptr logp;         /* out f32 [rows] (needs tokens), or 0 */
    nrl_devptr entropy;      /* out f32 [rows], or 0 */
    nrl_devptr rowstats;     /* out f32 [rows, 4], or 0 */
    nrl_devptr status;       /* out u8 [rows], or 0 */
    nrl_devptr logits_out;   /* out bf16 [rows, V], or 0 */
    nrl_devptr workspace;    /* scratch */
    uint64_t workspace_bytes;
    nrl_devptr allow_mask;   /* u8 allow-mask as in nrl_row_fwd ([rows, V], or [1, V] with stride 0), or 0 */
    uint64_t allow_row_stride; /* V or 0 */
    nrl_devptr uniforms;     /* f32 [rows] in [0,1), for NRL_READOUT_SAMPLE; else 0 */
    float temperature;       /* τ > 0: the logits are divided by it before they are folded (tempered_logits, src/nn/rl.rs:475-486;
                                `logits_out` keeps the undivided ones); 0 means 1 */
    uint32_t reserved;       /* 0 */
} nrl_readout_args;

/* scratch for a call with these flags (sampling adds 32 bytes per row and vocabulary tile). More than
 * 24 576 rows run as several launches of at most that many rows in stream order over the same scratch,
 * so it stops growing there. */
uint64_t nrl_readout_workspace_bytes(uint64_t rows, uint32_t V, uint32_t d, uint32_t flags);
int nrl_readout_fwd(const nrl_readout_args* args, nrl_stream stream);

/* check_scored_finite (src/nn/rl.rs:204-211), the check the reference's losses run in debug
 * builds (debug_check, :213-221, called from policy_gradient_loss :230, clipped_policy_loss
 * :268-269 and kl_estimate :386-387): every scored log-probability is finite. `logp` is f32 [n]
 * (n = S·B·T), `mask` the f32 scoring mask [n] or 0 (every position scored). One small kernel finds
 * the first flat position with mask != 0 whose value is not finite and leaves (position, value bits)
 * in `result`, 16 bytes of device memory of the caller's, 8-byte aligned; the call then reads
 * them back and synchronises the stream (the reference's check is a host read too). Returns NRL_OK
 * when there is none, else NRL_E_NOT_FINITE with *first_position and *value set; the wrapper
 * formats the reference's message "{what}: the scored log-probability at flat position {i} is
 * {value} (not finite)". A -inf there is a scored token the distribution excludes (a sampling
 * mask that was not applied to the training logits, or a token from elsewhere). */
int nrl_check_scored_finite(nrl_devptr logp, nrl_devptr mask, uint64_t n, nrl_devptr result, nrl_stream stream, uint64_t* first_position, float* value);

#ifdef __cplusplus
}
#endif
#endif /* NRL_H */
