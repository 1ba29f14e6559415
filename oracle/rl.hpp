// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of noetic-tensor's `nn::rl` (src/nn/rl.rs), op by op, on the engine restated in
// engine.hpp. Instantiated at float it follows `Cpu(Reference)` / `Cpu(Fast)` in f32; at double
// it is the F64 path the reference's own tests use as their truth. Each function cites the lines
// it follows. Only tests and the benchmark's CPU-baseline leg may use it.
#pragma once
#include "engine.hpp"

namespace orc {

// src/nn/rl.rs:36-55
enum class TokenReduction { None = 0, Sum = 1, TokenMean = 2, PerSequence = 3, SequenceMean = 4 };
// src/nn/rl.rs:356-364
enum class KlEstimator { K1 = 1, K2 = 2, K3 = 3 };

// src/nn/rl.rs:160-198
struct Clip {
    double low, high;
    bool has_dual;
    double dual;
    bool has_log_ratio_clamp;
    double log_ratio_clamp;
    void check() const {
        if (!(low >= 0.0 && low < 1.0 && high >= 0.0 && std::isfinite(low) && std::isfinite(high))) fail("clip range (need 0 <= low < 1, 0 <= high)");
        if (has_dual && !(dual > 1.0 && std::isfinite(dual))) fail("dual clip (need c > 1)");
        if (has_log_ratio_clamp && !(log_ratio_clamp > 0.0)) fail("log-ratio clamp (need b > 0)");
    }
};

template <class T>
struct Rl {
    typedef Engine<T> E;
    typedef typename E::Tensor Tensor;

    // src/nn/rl.rs:58-66
    static Tensor mask_or_ones(const Tensor* mask, const Tensor& like) {
        if (mask) {
            if (mask->sh != like.sh) fail("rl: mask shape");
            return mask->detach();
        }
        return Tensor::full(like.sh, 1.0);
    }

    // src/nn/rl.rs:88-92
    static Tensor per_sequence(const Tensor& per, const Tensor& mask) {
        size_t s = per.sh[0], b = per.sh[1];
        Tensor count = E::reshape(E::clamp_min(E::sum_dim(mask, 2), 1.0), {s, b});
        return E::div(E::reshape(E::sum_dim(per, 2), {s, b}), count);
    }

    // src/nn/rl.rs:69-86
    static Tensor reduce_tokens(const Tensor& per, const Tensor& mask, TokenReduction r) {
        size_t s = per.sh[0], b = per.sh[1], t = per.sh[2];
        switch (r) {
            case TokenReduction::None: return per;
            case TokenReduction::Sum: return E::reshape(E::sum_dim(E::reshape(per, {s, b * t}), 1), {s});
            case TokenReduction::TokenMean: {
                Tensor count = E::reshape(E::clamp_min(E::sum_dim(E::reshape(mask, {s, b * t}), 1), 1.0), {s});
                return E::div(E::reshape(E::sum_dim(E::reshape(per, {s, b * t}), 1), {s}), count);
            }
            case TokenReduction::PerSequence: return per_sequence(per, mask);
            case TokenReduction::SequenceMean: {
                Tensor seq = per_sequence(per, mask);
                Tensor nonempty = E::reshape(E::clamp_min(E::sum_dim(E::reshape(E::clamp_max(E::sum_dim(mask, 2), 1.0), {s, b}), 1), 1.0), {s});
                return E::div(E::reshape(E::sum_dim(seq, 1), {s}), nonempty);
            }
        }
        fail("reduction");
    }

    // src/nn/rl.rs:95-102
    static Bool masked_out(const Tensor& mask) { return E::equal_elem(mask, 0.0); }
    static Tensor zero_masked(const Tensor& x, const Tensor& mask) { return E::mask_fill(x, masked_out(mask), 0.0); }

    // src/nn/rl.rs:106-120
    static Tensor token_weights(const Tensor& w, const Tensor& like) {
        size_t s = like.sh[0], b = like.sh[1], t = like.sh[2];
        Tensor wd = w.detach();
        if (wd.rank() == 2) {
            if (wd.sh != Shape{s, b}) fail("per-sequence weights [S, B]");
            return E::reshape(wd, {s, b, 1});
        }
        if (wd.rank() == 3) {
            if (wd.sh != Shape{s, b, t}) fail("per-token weights [S, B, T]");
            return wd;
        }
        fail("weights rank");
    }

    // src/nn/rl.rs:124-129
    static Tensor select_max(const Tensor& a, const Tensor& b) {
        Tensor d = E::sub(a, b).untracked();
        Bool a_wins = E::greater_elem(d, 0.0);
        Bool b_wins = a_wins.bool_not();
        return E::add(E::mask_fill(a, b_wins, 0.0), E::mask_fill(b, a_wins, 0.0));
    }

    // src/nn/rl.rs:249-252
    static Tensor select(const Bool& pick, const Tensor& t, const Tensor& f) {
        Bool nt = pick.bool_not();
        return E::add(E::mask_fill(t, nt, 0.0), E::mask_fill(f, pick, 0.0));
    }

    // src/nn/rl.rs:134-141
    static Tensor token_log_probs(const Tensor& logits, const Int& tokens) {
        size_t r = logits.rank();
        if (r < 1) fail("token_log_probs: logits of rank 0");
        Shape lead(logits.sh.begin(), logits.sh.end() - 1);
        if (lead != tokens.sh) fail("token_log_probs: tokens shape");
        Tensor logp = E::log_softmax(logits, r - 1);
        Int idx = tokens;
        idx.sh.push_back(1);
        return E::reshape(E::gather(logp, r - 1, idx), tokens.sh);
    }

    // src/nn/rl.rs:228-235
    static Tensor policy_gradient_loss(const Tensor& logp, const Tensor& weights, const Tensor* mask, TokenReduction r) {
        if (logp.rank() != 3) fail("policy_gradient_loss: logp [S, B, T]");
        Tensor m = mask_or_ones(mask, logp);
        Tensor w = token_weights(weights, logp);
        Tensor per = zero_masked(E::neg(E::mul(logp, w)), m);
        return reduce_tokens(per, m, r);
    }

    // src/nn/rl.rs:239-246
    static Tensor log_ratio(const Tensor& logp, const Tensor& old_logp, const Tensor& m, bool has_clamp, double b) {
        if (old_logp.sh != logp.sh) fail("rl: old log-probabilities shape");
        Tensor d = zero_masked(E::sub(logp, old_logp.detach()), m);
        return has_clamp ? E::clamp(d, -b, b) : d;
    }

    // src/nn/rl.rs:265-287
    static Tensor clipped_policy_loss(const Tensor& logp, const Tensor& old_logp, const Tensor& advantages, const Tensor* mask, Clip clip, TokenReduction red) {
        clip.check();
        if (logp.rank() != 3) fail("clipped_policy_loss: logp [S, B, T]");
        Tensor m = mask_or_ones(mask, logp);
        Tensor a = token_weights(advantages, logp);
        Tensor r = E::exp(log_ratio(logp, old_logp, m, clip.has_log_ratio_clamp, clip.log_ratio_clamp));
        Tensor unclipped = E::neg(E::mul(r, a));
        Tensor clipped = E::neg(E::mul(E::clamp(r, 1.0 - clip.low, 1.0 + clip.high), a));
        Tensor ppo = select_max(unclipped, clipped);
        Tensor per = ppo;
        if (clip.has_dual) {
            Tensor ae = E::expand(a, ppo.sh);
            Tensor cap = E::mul_scalar(ae, -clip.dual);
            Tensor capped = E::neg(select_max(E::neg(ppo), E::neg(cap)));
            per = select(E::lower_elem(ae.untracked(), 0.0), capped, ppo);
        }
        return reduce_tokens(zero_masked(per, m), m, red);
    }

    // src/nn/rl.rs:293-317
    static Tensor clip_fraction(const Tensor& logp_in, const Tensor& old_logp, const Tensor& advantages, const Tensor* mask, Clip clip) {
        clip.check();
        Tensor logp = logp_in.detach();
        Tensor m = mask_or_ones(mask, logp);
        Tensor a = token_weights(advantages, logp);
        Tensor d = log_ratio(logp, old_logp, m, false, 0.0);
        Tensor r = E::exp(d);
        size_t s = r.sh[0], b = r.sh[1], t = r.sh[2];
        auto f = [](const Bool& x) { return E::float_of(x); };
        Tensor pos = f(E::greater_elem(a, 0.0));
        Tensor ng = f(E::lower_elem(a, 0.0));
        Tensor up = f(E::greater_elem(r, 1.0 + clip.high));
        Tensor down = f(E::lower_elem(r, 1.0 - clip.low));
        Tensor hit = E::add(E::mul(up, pos), E::mul(down, ng));
        if (clip.has_dual) hit = E::add(hit, E::mul(f(E::greater_elem(r, clip.dual)), ng));
        if (clip.has_log_ratio_clamp) hit = E::add(hit, f(E::greater_elem(E::abs(d), clip.log_ratio_clamp)));
        hit = E::mul(E::clamp_max(hit, 1.0), m);
        Tensor count = E::reshape(E::clamp_min(E::sum_dim(E::reshape(m, {s, b * t}), 1), 1.0), {s});
        return E::div(E::reshape(E::sum_dim(E::reshape(hit, {s, b * t}), 1), {s}), count);
    }

    // src/nn/rl.rs:327-338
    static Tensor categorical_kl(const Tensor& logits, const Tensor& ref_logits, const Tensor* mask, TokenReduction red) {
        if (logits.rank() != 4) fail("categorical_kl: logits [S, B, T, V]");
        if (logits.sh != ref_logits.sh) fail("categorical_kl: reference logits shape");
        size_t s = logits.sh[0], b = logits.sh[1], t = logits.sh[2];
        Tensor logp = E::log_softmax(logits, 3);
        Tensor logr = E::log_softmax(ref_logits.detach(), 3);
        Bool zero_p = E::equal_elem(logp.untracked(), -std::numeric_limits<double>::infinity());
        Tensor diff = E::mask_fill(E::sub(logp, logr), zero_p, 0.0);
        Tensor per = E::reshape(E::sum_dim(E::mul(E::exp(logp), diff), 3), {s, b, t});
        Tensor m = mask_or_ones(mask, per);
        return reduce_tokens(zero_masked(per, m), m, red);
    }

    // src/nn/rl.rs:475-486
    static Tensor tempered_logits(const Tensor& logits, double temperature, const Tensor* mask) {
        if (!(temperature > 0.0 && std::isfinite(temperature))) fail("tempered_logits: temperature must be positive");
        Tensor z = temperature == 1.0 ? logits : E::div_scalar(logits, temperature);
        if (mask) {
            if (mask->rank() != z.rank()) fail("tempered_logits: mask rank");
            return E::add(z, mask->detach());
        }
        return z;
    }

    // src/nn/rl.rs:347-351
    static Tensor reference_kl(const Tensor& logits, const Tensor& ref_logits, double temperature, const Tensor* vocab_mask, const Tensor* mask, TokenReduction red) {
        Tensor p = tempered_logits(logits, temperature, vocab_mask);
        Tensor r = tempered_logits(ref_logits.detach(), temperature, vocab_mask);
        return categorical_kl(p, r, mask, red);
    }

    // src/nn/rl.rs:380-400
    static Tensor kl_estimate(const Tensor& logp, const Tensor& ref_logp, KlEstimator e, bool has_clamp, double b, const Tensor* mask, TokenReduction red) {
        if (logp.rank() != 3) fail("kl_estimate: logp [S, B, T]");
        if (logp.sh != ref_logp.sh) fail("kl_estimate: reference log-probabilities shape");
        if (has_clamp && !(b > 0.0)) fail("kl_estimate: delta clamp (need b > 0)");
        Tensor m = mask_or_ones(mask, logp);
        Tensor delta = zero_masked(E::sub(ref_logp.detach(), logp), m);
        if (has_clamp) delta = E::clamp(delta, -b, b);
        Tensor per;
        switch (e) {
            case KlEstimator::K1: per = E::neg(delta); break;
            case KlEstimator::K2: per = E::div_scalar(E::mul(delta, delta), 2.0); break;
            case KlEstimator::K3: per = E::sub(E::exp(delta), E::add_scalar(delta, 1.0)); break;
        }
        return reduce_tokens(zero_masked(per, m), m, red);
    }

    // src/nn/rl.rs:405-414
    static Tensor categorical_entropy(const Tensor& logits, const Tensor* mask, TokenReduction red) {
        if (logits.rank() != 4) fail("categorical_entropy: logits [S, B, T, V]");
        size_t s = logits.sh[0], b = logits.sh[1], t = logits.sh[2];
        Tensor logp = E::log_softmax(logits, 3);
        Bool zero_p = E::equal_elem(logp.untracked(), -std::numeric_limits<double>::infinity());
        Tensor safe = E::mask_fill(logp, zero_p, 0.0);
        Tensor per = E::reshape(E::neg(E::sum_dim(E::mul(E::exp(logp), safe), 3)), {s, b, t});
        Tensor m = mask_or_ones(mask, per);
        return reduce_tokens(zero_masked(per, m), m, red);
    }
};

// src/nn/rl.rs:436-461 (host f64 whatever the tensor dtype)
inline std::vector<double> group_advantages(const double* rewards, size_t len, size_t n, int norm_std, double eps, bool unbiased) {
    if (!(n >= 1 && len % n == 0)) fail("group_advantages: rewards in groups of n");
    if (norm_std) {
        if (!(eps >= 0.0)) fail("group_advantages: eps < 0");
        if (unbiased && n < 2) fail("group_advantages: the sample standard deviation needs groups of at least 2");
    }
    std::vector<double> out;
    out.reserve(len);
    for (size_t g0 = 0; g0 < len; g0 += n) {
        const double* g = rewards + g0;
        double lo = std::numeric_limits<double>::infinity(), hi = -lo;
        for (size_t i = 0; i < n; i++) {
            lo = std::fmin(lo, g[i]);
            hi = std::fmax(hi, g[i]);
        }
        if (lo == hi) {
            for (size_t i = 0; i < n; i++) out.push_back(0.0);
            continue;
        }
        double sum = 0.0;
        for (size_t i = 0; i < n; i++) sum += g[i];
        double mean = sum / (double)n;
        double scale = 1.0;
        if (norm_std) {
            double ss = 0.0;
            for (size_t i = 0; i < n; i++) ss += (g[i] - mean) * (g[i] - mean);
            double var = ss / (unbiased ? (double)(n - 1) : (double)n);
            scale = std::sqrt(var) + eps;
        }
        for (size_t i = 0; i < n; i++) out.push_back((g[i] - mean) / scale);
    }
    return out;
}

}  // namespace orc
