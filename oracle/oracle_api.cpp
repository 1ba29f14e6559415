// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// Flat C entry points over the CPU restatement (engine.hpp, rl.hpp, streams.hpp), loaded with
// ctypes by tests/ and by the benchmark's CPU-baseline / reference legs. The shipped library
// never links or calls this file.
#include "oracle.h"
#include "loss.hpp"
#include "rl.hpp"
#include "streams.hpp"

#include <algorithm>
#include <cstring>

using namespace orc;

static thread_local std::string g_err;

extern "C" const char* orc_last_error(void) { return g_err.c_str(); }

extern "C" int orc_set_backend(int fast, int threads) {
    config().mode = fast ? CpuMode::Fast : CpuMode::Reference;
    config().threads = threads < 1 ? 1 : threads;
    return 0;
}

// Values of `dtype`-typed storage as the engine's T: f32 as is, bf16 upcast exactly
// (src/tensor/float.rs:92-100), f64 cast as `from_f64s` does.
template <class T>
static std::vector<T> load(const void* p, int dtype, size_t n) {
    std::vector<T> v(n);
    switch (dtype) {
        case ORC_F32: { const float* s = (const float*)p; for (size_t i = 0; i < n; i++) v[i] = (T)s[i]; break; }
        case ORC_F64: { const double* s = (const double*)p; for (size_t i = 0; i < n; i++) v[i] = (T)s[i]; break; }
        case ORC_BF16: { const uint16_t* s = (const uint16_t*)p; for (size_t i = 0; i < n; i++) v[i] = (T)bf16_to_f32(s[i]); break; }
        default: fail("unknown storage dtype");
    }
    return v;
}

template <class T>
static int eval(const orc_rl_case* c) {
    typedef Engine<T> E;
    typedef Rl<T> R;
    typedef typename E::Tensor Tensor;
    size_t S = c->S, B = c->B, Tn = c->T, V = c->V, n = S * B * Tn;
    Shape tok_sh{S, B, Tn}, lsh{S, B, Tn, V};
    auto small = [&](const double* p, Shape sh) { return Tensor::from_f64s(p, sh); };

    Tensor leaf;      // the tensor the gradient is taken of
    Tensor logp;      // [S,B,T] log-probabilities entering the token-level losses
    Tensor logits;
    std::optional<Tensor> vmask;
    if (c->vocab_mask) vmask = c->vocab_mask_full ? small(c->vocab_mask, lsh) : small(c->vocab_mask, Shape{1, 1, 1, V});
    bool needs_logits = c->logits != nullptr;
    if (needs_logits) {
        logits = Tensor(load<T>(c->logits, c->logits_dtype, n * V), lsh);
        if (c->upstream) logits = logits.require_grad();
        leaf = logits;
    }
    Int tokens;
    if (c->tokens) {
        tokens.v.assign(c->tokens, c->tokens + n);
        tokens.sh = tok_sh;
    }
    auto tempered = [&](const Tensor& x) { return (c->temperature != 1.0 || vmask) ? R::tempered_logits(x, c->temperature, vmask ? &*vmask : nullptr) : x; };
    if (c->logp) {
        logp = small(c->logp, tok_sh);
        if (c->upstream) logp = logp.require_grad();
        leaf = logp;
    } else if (needs_logits && c->tokens && c->op < ORC_OP_NLL) {
        logp = R::token_log_probs(tempered(logits), tokens);
    }
    std::optional<Tensor> mask, old_logp, ref_logp, weights, ref_logits;
    if (c->mask) mask = small(c->mask, tok_sh);
    if (c->old_logp) old_logp = small(c->old_logp, tok_sh);
    if (c->ref_logp) ref_logp = small(c->ref_logp, tok_sh);
    if (c->weights) weights = c->weights_rank == 2 ? small(c->weights, Shape{S, B}) : small(c->weights, tok_sh);
    if (c->ref_logits) ref_logits = Tensor(load<T>(c->ref_logits, c->ref_dtype, n * V), lsh);
    if (ref_logits && c->out_grad_ref && c->upstream) ref_logits = ref_logits->require_grad();
    const Tensor* mp = mask ? &*mask : nullptr;
    TokenReduction red = (TokenReduction)c->reduction;
    Clip clip{c->clip_low, c->clip_high, c->has_dual != 0, c->dual, c->has_log_ratio_clamp != 0, c->log_ratio_clamp};

    Tensor out;
    switch (c->op) {
        case ORC_OP_TOKEN_LOG_PROBS:
            out = logp;
            // The reference's device test zeroes masked positions of the raw log-probabilities
            // (src/nn/tests/gpu/rl.rs:81) so that −∞ entries do not enter the comparison.
            if (mp) out = E::mask_fill(out, E::equal_elem(*mp, 0.0), 0.0);
            break;
        case ORC_OP_PG: out = R::policy_gradient_loss(logp, *weights, mp, red); break;
        case ORC_OP_PPO: out = R::clipped_policy_loss(logp, *old_logp, *weights, mp, clip, red); break;
        case ORC_OP_CLIP_FRACTION: out = R::clip_fraction(logp, *old_logp, *weights, mp, clip); break;
        case ORC_OP_KL: out = R::categorical_kl(logits, *ref_logits, mp, red); break;
        case ORC_OP_REFERENCE_KL: out = R::reference_kl(logits, *ref_logits, c->temperature, vmask ? &*vmask : nullptr, mp, red); break;
        case ORC_OP_KL_ESTIMATE: out = R::kl_estimate(logp, *ref_logp, (KlEstimator)c->estimator, c->has_delta_clamp != 0, c->delta_clamp, mp, red); break;
        case ORC_OP_ENTROPY: out = R::categorical_entropy(tempered(logits), mp, red); break;
        case ORC_OP_NLL: out = Loss<T>::nll(logits, tokens); break;
        case ORC_OP_CE: out = Loss<T>::cross_entropy(logits, tokens); break;
        case ORC_OP_MASKED_CE: out = Loss<T>::masked_cross_entropy(logits, tokens, *mask); break;
        case ORC_OP_CE_WITH: {
            CeOptions o;
            o.has_ignore_index = c->has_ignore_index != 0;
            o.ignore_index = c->ignore_index;
            o.smoothing = c->smoothing;
            out = Loss<T>::cross_entropy_with(logits, tokens, mp, o);
            break;
        }
        case ORC_OP_KL_DIV: out = Loss<T>::kl_div(logits, *ref_logits); break;
        default: fail("unknown op");
    }
    if ((int64_t)out.n() > c->out_capacity) fail("output buffer too small");
    for (size_t i = 0; i < out.n(); i++) c->out_value[i] = (double)out.v()[i];
    *c->out_len = (int64_t)out.n();
    if (c->upstream && c->out_grad) {
        // (l * up).sum().backward(), as src/nn/tests/gpu/rl.rs:98-102
        Tensor up = small(c->upstream, out.sh);
        Tensor root = E::sum(E::mul(out, up));
        auto g = E::backward(root);
        const Tensor* gl = g.get(leaf);
        size_t ln = leaf.n();
        if (!gl) {
            for (size_t i = 0; i < ln; i++) c->out_grad[i] = 0.0;
        } else {
            for (size_t i = 0; i < ln; i++) c->out_grad[i] = (double)gl->v()[i];
        }
        if (c->out_grad_ref && ref_logits) {
            const Tensor* gr = g.get(*ref_logits);
            for (size_t i = 0; i < ref_logits->n(); i++) c->out_grad_ref[i] = gr ? (double)gr->v()[i] : 0.0;
        }
    }
    return 0;
}

extern "C" int orc_rl_eval(const orc_rl_case* c) {
    try {
        if (c->struct_size != sizeof(orc_rl_case)) fail("orc_rl_case: struct size mismatch");
        return c->engine_dtype == ORC_F64 ? eval<double>(c) : eval<float>(c);
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

template <class T>
static void lane_op(int op, const void* x, int x_dtype, size_t rows, size_t V, const double* upstream, double* out_value, int64_t* out_index, double* out_grad) {
    typedef Engine<T> E;
    typedef typename E::Tensor Tensor;
    Tensor leaf(load<T>(x, x_dtype, rows * V), Shape{rows, V});
    if (op == 3) {
        auto am = E::argmax(leaf, 1);
        for (size_t r = 0; r < rows; r++) {
            out_index[r] = am.v[r];
            if (out_value) out_value[r] = (double)leaf.v()[r * V + (size_t)am.v[r]];
        }
        return;
    }
    if (upstream) leaf = leaf.require_grad();
    Tensor out;
    switch (op) {
        case 0: out = E::softmax(leaf, 1); break;
        case 1: out = E::log_softmax(leaf, 1); break;
        case 2: out = E::logsumexp(leaf, 1); break;
        case 4: out = E::sum_dim(leaf, 1); break;
        default: fail("orc_lane_op: unknown op");
    }
    for (size_t i = 0; i < out.n(); i++) out_value[i] = (double)out.v()[i];
    if (upstream) {
        Tensor up = Tensor::from_f64s(upstream, out.sh);
        auto g = E::backward(E::sum(E::mul(out, up)));
        const Tensor* gl = g.get(leaf);
        for (size_t i = 0; i < rows * V; i++) out_grad[i] = gl ? (double)gl->v()[i] : 0.0;
    }
}

extern "C" int orc_lane_op(int op, int engine_dtype, const void* x, int x_dtype, int64_t rows, int64_t V, const double* upstream, double* out_value,
                           int64_t* out_index, double* out_grad) {
    try {
        if (engine_dtype == ORC_F64) lane_op<double>(op, x, x_dtype, (size_t)rows, (size_t)V, upstream, out_value, out_index, out_grad);
        else lane_op<float>(op, x, x_dtype, (size_t)rows, (size_t)V, upstream, out_value, out_index, out_grad);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// check_scored_finite (src/nn/rl.rs:204-211): `(0..v.len()).find(|&i| m.is_none_or(|m| m[i] != 0.0) && !v[i].is_finite())`.
extern "C" int64_t orc_check_scored_finite(const double* logp, const double* mask, int64_t n) {
    for (int64_t i = 0; i < n; i++)
        if ((!mask || mask[i] != 0.0) && !std::isfinite(logp[i])) return i;
    return -1;
}

extern "C" int orc_group_advantages(const double* rewards, int64_t len, int64_t n, int norm_std, double eps, int unbiased, double* out) {
    try {
        auto v = group_advantages(rewards, (size_t)len, (size_t)n, norm_std, eps, unbiased != 0);
        std::copy(v.begin(), v.end(), out);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// ------------------------------------------------------------------------------ streams

extern "C" void orc_sha256(const void* data, int64_t n, uint8_t out[32]) {
    Sha256 h;
    h.update(data, (size_t)n);
    h.finish(out);
}

extern "C" void orc_chacha20_words(const uint8_t seed[32], int64_t skip_words, int64_t n, uint32_t* out) {
    ChaCha20Rng r(seed);
    for (int64_t i = 0; i < skip_words; i++) r.next_u32();
    for (int64_t i = 0; i < n; i++) out[i] = r.next_u32();
}

extern "C" void orc_derive_seed(uint64_t root, const char* label, uint8_t seed[32]) {
    Sha256 h;
    uint8_t le[8];
    for (int i = 0; i < 8; i++) le[i] = (uint8_t)(root >> (8 * i));
    h.update(le, 8);
    h.update(label, std::strlen(label));
    h.finish(seed);
}

// One f32 uniform on [0,1) per row, from the derived stream in row-major order:
// (next_u32() >> 8) · 2^-24. This is the build's own convention for the caller-supplied uniforms
// of the inverse-CDF sampler (the reference's sampler draws Gumbel noise per logit instead).
extern "C" void orc_row_uniforms(uint64_t root, const char* label, int64_t rows, float* out) {
    ChaCha20Rng r = ChaCha20Rng::derive(root, label);
    for (int64_t i = 0; i < rows; i++) out[i] = (float)(r.next_u32() >> 8) * (1.0f / 16777216.0f);
}

extern "C" void orc_bf16_from_f32(const float* x, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; i++) out[i] = bf16_from_f32(x[i]);
}
extern "C" void orc_bf16_to_f32(const uint16_t* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = bf16_to_f32(x[i]);
}

// ------------------------------------------------------------------------------ samplers

// z = logits / τ + mask in f32, as `tempered_logits` (src/nn/rl.rs:475-486) leaves it; an
// allow-mask byte of 0 is the additive −∞.
static void tempered_row(const void* logits, int dtype, size_t row, size_t V, float tau, const float* add_mask, size_t add_stride, const uint8_t* allow, size_t allow_stride, std::vector<float>& z) {
    z.resize(V);
    for (size_t v = 0; v < V; v++) {
        float x;
        switch (dtype) {
            case ORC_F32: x = ((const float*)logits)[row * V + v]; break;
            case ORC_BF16: x = bf16_to_f32(((const uint16_t*)logits)[row * V + v]); break;
            default: x = (float)((const double*)logits)[row * V + v];
        }
        if (tau != 1.0f) x = x / tau;
        if (add_mask) x = x + add_mask[row * add_stride + v];
        if (allow && !allow[row * allow_stride + v]) x = -std::numeric_limits<float>::infinity();
        z[v] = x;
    }
}

// The reference's sampler (src/nn/rl.rs:490-529): Gumbel-max with one ChaCha20 `next_u64` per
// logit in row-major order, noise computed in f64, cast to f32, added in f32, first-max argmax.
// temperature 0 is the argmax of the masked logits and draws nothing. Returns -2 and the row in
// *bad_row when a row has no allowed token or a NaN (the reference panics there).
extern "C" int orc_sample_gumbel(const void* logits, int dtype, int64_t rows, int64_t V, double temperature, const float* add_mask, int64_t add_stride,
                                 const uint8_t* allow, int64_t allow_stride, uint64_t root, const char* label, int64_t* tokens, int64_t* bad_row) {
    ChaCha20Rng rng = ChaCha20Rng::derive(root, label);
    float tau = temperature == 0.0 ? 1.0f : (float)temperature;
    std::vector<float> z;
    std::vector<std::vector<float>> all((size_t)rows);
    for (int64_t r = 0; r < rows; r++) {
        tempered_row(logits, dtype, (size_t)r, (size_t)V, tau, add_mask, (size_t)add_stride, allow, (size_t)allow_stride, z);
        auto am = Engine<float>::argmax_dim(z, Shape{(size_t)V}, 0);
        float top = z[(size_t)am.first[0]];
        if (top != top || top == -std::numeric_limits<float>::infinity()) {
            if (bad_row) *bad_row = r;
            g_err = "sample_categorical: position has no allowed token (every logit -inf or a NaN)";
            return -2;
        }
        all[(size_t)r] = z;
    }
    for (int64_t r = 0; r < rows; r++) {
        std::vector<float>& zr = all[(size_t)r];
        if (temperature != 0.0) {
            for (int64_t v = 0; v < V; v++) {
                uint64_t k = rng.next_u64() >> 11;
                double u = ((double)k + 0.5) / 9007199254740992.0;
                float g = (float)(-std::log(-std::log(u)));
                zr[(size_t)v] = zr[(size_t)v] + g;
            }
        }
        tokens[r] = Engine<float>::argmax_dim(zr, Shape{(size_t)V}, 0).first[0];
    }
    return 0;
}

// The inverse-CDF sampler the B200 path implements, evaluated in f64 on the f32 tempered logits:
//   m = max over allowed z;  e_v = exp(z_v − m) (0 where excluded);  Z = Σ e_v;  t = u·Z;
//   token = min{k : Σ_{v≤k} e_v > t}  (index order).
// Also per row, in f64: log-prob of the token, entropy, and (with reference logits, tempered and
// masked the same way) the exact KL and the token's reference log-prob. A row is a *boundary* row
// when t lies within 1e-6·Z of the cumulative sum just below or just above the chosen token (the
// lower one only if an earlier token has mass): there an f32 evaluation may legitimately pick a
// neighbour. status bit0: no allowed token; bit1: NaN.
// PARITY UNPINNED for the sampled tokens: the reference has no inverse-CDF sampler (its own is
// Gumbel-max, restated above), so this function is the definition, not a restatement. The values
// it returns beside the token (log-prob, KL, entropy) are checked in the tests against the
// restated engine's token_log_probs / reference_kl / categorical_entropy, which are pinned.
extern "C" int orc_sample_inverse_cdf(const void* logits, int dtype, const void* ref_logits, int ref_dtype, int64_t rows, int64_t V, double temperature,
                                      const float* add_mask, int64_t add_stride, const uint8_t* allow, int64_t allow_stride, const float* uniforms,
                                      const int64_t* given_tokens, int64_t* tokens, uint8_t* boundary, double* logp, double* ref_logp, double* kl,
                                      double* entropy, uint8_t* status) {
    float tau = temperature == 0.0 ? 1.0f : (float)temperature;
    const double ninf = -std::numeric_limits<double>::infinity();
    std::vector<float> z, zr;
    std::vector<double> e((size_t)V);
    for (int64_t r = 0; r < rows; r++) {
        tempered_row(logits, dtype, (size_t)r, (size_t)V, tau, add_mask, (size_t)add_stride, allow, (size_t)allow_stride, z);
        if (ref_logits) tempered_row(ref_logits, ref_dtype, (size_t)r, (size_t)V, tau, add_mask, (size_t)add_stride, allow, (size_t)allow_stride, zr);
        double m = ninf;
        bool nan = false;
        for (int64_t v = 0; v < V; v++) {
            if (z[(size_t)v] != z[(size_t)v]) nan = true;
            m = std::max(m, (double)z[(size_t)v]);
        }
        uint8_t st = 0;
        if (nan) st |= 2;
        if (!nan && m == ninf) st |= 1;
        if (status) status[r] = st;
        if (st) {
            if (tokens) tokens[r] = -1;
            if (boundary) boundary[r] = 0;
            double q = std::numeric_limits<double>::quiet_NaN();
            if (logp) logp[r] = q;
            if (ref_logp) ref_logp[r] = q;
            if (kl) kl[r] = q;
            if (entropy) entropy[r] = q;
            continue;
        }
        double Z = 0.0;
        for (int64_t v = 0; v < V; v++) {
            e[(size_t)v] = std::exp((double)z[(size_t)v] - m);
            Z += e[(size_t)v];
        }
        int64_t tok = -1;
        uint8_t bnd = 0;
        if (given_tokens) {
            tok = given_tokens[r];
        } else if (temperature == 0.0) {
            tok = Engine<float>::argmax_dim(z, Shape{(size_t)V}, 0).first[0];
        } else {
            double t = (double)uniforms[r] * Z;
            double c = 0.0, prev = 0.0;
            int64_t last_pos = -1;
            for (int64_t v = 0; v < V; v++) {
                if (e[(size_t)v] > 0.0) last_pos = v;
                double nc = c + e[(size_t)v];
                if (nc > t) {
                    tok = v;
                    prev = c;
                    c = nc;
                    break;
                }
                c = nc;
            }
            if (tok < 0) {  // t ≥ Σ (rounding only): the last token with mass
                tok = last_pos;
                bnd = 1;
            } else {
                if (c - t <= 1e-6 * Z) bnd = 1;
                if (prev > 0.0 && t - prev <= 1e-6 * Z) bnd = 1;
            }
        }
        if (tokens) tokens[r] = tok;
        if (boundary) boundary[r] = bnd;
        double lnZ = std::log(Z);
        if (logp) logp[r] = ((double)z[(size_t)tok] - m) - lnZ;
        if (entropy) {
            double h = 0.0;
            for (int64_t v = 0; v < V; v++) {
                double lp = ((double)z[(size_t)v] - m) - lnZ;
                if (lp != ninf) h += std::exp(lp) * lp;
            }
            entropy[r] = -h;
        }
        if (ref_logits) {
            double mr = ninf;
            for (int64_t v = 0; v < V; v++) mr = std::max(mr, (double)zr[(size_t)v]);
            double Zr = 0.0;
            for (int64_t v = 0; v < V; v++) Zr += std::exp((double)zr[(size_t)v] - mr);
            double lnZr = std::log(Zr);
            if (ref_logp) ref_logp[r] = ((double)zr[(size_t)tok] - mr) - lnZr;
            if (kl) {
                double k = 0.0;
                for (int64_t v = 0; v < V; v++) {
                    double lp = ((double)z[(size_t)v] - m) - lnZ;
                    if (lp == ninf) continue;
                    double lr = ((double)zr[(size_t)v] - mr) - lnZr;
                    k += std::exp(lp) * (lp - lr);
                }
                kl[r] = k;
            }
        }
    }
    return 0;
}
