/* TEST INFRASTRUCTURE — NOT PRODUCT CODE.
 *
 * C interface of the CPU restatement of noetic-tensor's `nn::rl` path (see engine.hpp, rl.hpp,
 * streams.hpp for the reference lines each part follows). Loaded with ctypes by tests/ and by the
 * benchmark's CPU-baseline and reference legs only.
 */
#ifndef NOETIC_RL_ORACLE_H
#define NOETIC_RL_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F32 = 0, ORC_F64 = 1, ORC_BF16 = 2 };

enum {
    ORC_OP_TOKEN_LOG_PROBS = 0, /* token_log_probs            src/nn/rl.rs:134-141 */
    ORC_OP_PG = 1,              /* policy_gradient_loss       src/nn/rl.rs:228-235 */
    ORC_OP_PPO = 2,             /* clipped_policy_loss        src/nn/rl.rs:265-287 */
    ORC_OP_CLIP_FRACTION = 3,   /* clip_fraction              src/nn/rl.rs:293-317 */
    ORC_OP_KL = 4,              /* categorical_kl             src/nn/rl.rs:327-338 */
    ORC_OP_REFERENCE_KL = 5,    /* reference_kl               src/nn/rl.rs:347-351 */
    ORC_OP_KL_ESTIMATE = 6,     /* kl_estimate                src/nn/rl.rs:380-400 */
    ORC_OP_ENTROPY = 7,         /* categorical_entropy        src/nn/rl.rs:405-414 */
    ORC_OP_NLL = 8,             /* nn::loss::nll              src/nn/loss.rs:10-16   -> [S, B·T] */
    ORC_OP_CE = 9,              /* cross_entropy              src/nn/loss.rs:19-22   -> [S] */
    ORC_OP_MASKED_CE = 10,      /* masked_cross_entropy       src/nn/loss.rs:27-34   -> [S] */
    ORC_OP_CE_WITH = 11,        /* cross_entropy_with         src/nn/loss.rs:48-79   -> [S] */
    ORC_OP_KL_DIV = 12          /* kl_div(pred = logits, target = ref_logits) src/nn/loss.rs:175-183 -> [S] */
};

/* One evaluation of an rl function and, with `upstream`, of the gradient of
 * sum(value * upstream) with respect to the leaf: the logits when `logits` is given and `logp` is
 * not, else `logp`. Small arrays are f64 and converted as the reference's `from_f64s` does. */
typedef struct orc_rl_case {
    uint32_t struct_size;
    int32_t op;
    int32_t engine_dtype; /* ORC_F32: Cpu(Reference)/Cpu(Fast) arithmetic; ORC_F64: the tests' truth */
    int32_t reduction;    /* 0 None, 1 Sum, 2 TokenMean, 3 PerSequence, 4 SequenceMean */
    int64_t S, B, T, V;
    const void* logits; /* [S,B,T,V] or NULL */
    int32_t logits_dtype;
    int32_t ref_dtype;
    const void* ref_logits;   /* [S,B,T,V] or NULL */
    const int64_t* tokens;    /* [S,B,T] or NULL */
    const double* logp;       /* [S,B,T] leaf log-probabilities, or NULL to take them from logits+tokens */
    const double* old_logp;   /* [S,B,T] */
    const double* ref_logp;   /* [S,B,T] */
    const double* weights;    /* weights / advantages, [S,B] or [S,B,T] */
    int32_t weights_rank;     /* 2 or 3 */
    int32_t estimator;        /* 1, 2, 3 */
    const double* mask;       /* scoring mask [S,B,T] of 0/1, or NULL */
    const double* vocab_mask; /* additive [V] (broadcast [1,1,1,V]), or NULL */
    double temperature;       /* 1.0 leaves the logits as they are */
    double clip_low, clip_high, dual, log_ratio_clamp, delta_clamp;
    int32_t has_dual, has_log_ratio_clamp, has_delta_clamp;
    int32_t vocab_mask_full; /* 1: vocab_mask is [S,B,T,V] (a per-position vocabulary mask) */
    const double* upstream; /* shape of the value, or NULL for no backward */
    double* out_value;
    int64_t out_capacity;
    int64_t* out_len;
    double* out_grad; /* leaf-shaped, or NULL */
    /* the cross-entropy family (ops 8-12); `tokens` are the targets */
    int32_t has_ignore_index;
    int32_t reserved0;
    int64_t ignore_index;
    double smoothing;
    double* out_grad_ref; /* ORC_OP_KL_DIV: gradient w.r.t. ref_logits (the target side), or NULL */
} orc_rl_case;

const char* orc_last_error(void);
int orc_set_backend(int fast, int threads);
int orc_rl_eval(const orc_rl_case* c);
/* check_scored_finite (src/nn/rl.rs:204-211): the first flat position whose mask (NULL = every
 * position scored) is non-zero and whose log-probability is not finite, or -1. */
int64_t orc_check_scored_finite(const double* logp, const double* mask, int64_t n);
int orc_group_advantages(const double* rewards, int64_t len, int64_t n, int norm_std, double eps, int unbiased, double* out);

void orc_sha256(const void* data, int64_t n, uint8_t out[32]);
void orc_chacha20_words(const uint8_t seed[32], int64_t skip_words, int64_t n, uint32_t* out);
void orc_derive_seed(uint64_t root, const char* label, uint8_t seed[32]);
void orc_row_uniforms(uint64_t root, const char* label, int64_t rows, float* out);
void orc_bf16_from_f32(const float* x, int64_t n, uint16_t* out);
void orc_bf16_to_f32(const uint16_t* x, int64_t n, float* out);

/* Lane operations of the tensor engine on a [rows, V] input (src/tensor/activation.rs:15-42, 71-77;
 * src/tensor/kernels.rs:122-209). op: 0 softmax, 1 log_softmax, 2 logsumexp (value [rows]),
 * 3 argmax (index in out_index, value in out_value[rows]), 4 sum_dim (value [rows]). With
 * `upstream` (shape of the value; ops 0-2) out_grad [rows, V] is d sum(value·upstream) / dx. */
int orc_lane_op(int op, int engine_dtype, const void* x, int x_dtype, int64_t rows, int64_t V, const double* upstream, double* out_value,
                int64_t* out_index, double* out_grad);

int orc_sample_gumbel(const void* logits, int dtype, int64_t rows, int64_t V, double temperature, const float* add_mask, int64_t add_stride,
                      const uint8_t* allow, int64_t allow_stride, uint64_t root, const char* label, int64_t* tokens, int64_t* bad_row);

int orc_sample_inverse_cdf(const void* logits, int dtype, const void* ref_logits, int ref_dtype, int64_t rows, int64_t V, double temperature,
                           const float* add_mask, int64_t add_stride, const uint8_t* allow, int64_t allow_stride, const float* uniforms,
                           const int64_t* given_tokens, int64_t* tokens, uint8_t* boundary, double* logp, double* ref_logp, double* kl,
                           double* entropy, uint8_t* status);

#ifdef __cplusplus
}
#endif
#endif
