// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of the cross-entropy family of noetic-tensor's `nn::loss` (src/nn/loss.rs),
// op by op on the engine of engine.hpp: the same log_softmax → one-hot product → negated lane
// sum order, the same product with the mask. Only tests and the benchmark's CPU legs use it.
#pragma once
#include "engine.hpp"

namespace orc {

// src/nn/loss.rs:36-43
struct CeOptions {
    bool has_ignore_index = false;
    int64_t ignore_index = 0;
    double smoothing = 0.0;
    bool is_default() const { return !has_ignore_index && smoothing == 0.0; }
};

template <class T>
struct Loss {
    typedef Engine<T> E;
    typedef typename E::Tensor Tensor;

    // src/nn/loss.rs:10-16: [S,B,T,V], [S,B,T] → [S, B·T]
    static Tensor nll(const Tensor& logits, const Int& targets) {
        if (logits.rank() != 4) fail("nll: logits [S, B, T, V]");
        size_t s = logits.sh[0], n = logits.sh[1] * logits.sh[2], v = logits.sh[3];
        Tensor logp = E::reshape(E::log_softmax(logits, 3), {s, n, v});
        Tensor onehot = E::one_hot(Int{targets.v, Shape{s, n}}, v);
        return E::neg(E::reshape(E::sum_dim(E::mul(logp, onehot), 2), {s, n}));
    }

    // src/nn/loss.rs:19-22
    static Tensor cross_entropy(const Tensor& logits, const Int& targets) {
        size_t s = logits.sh[0];
        return E::reshape(E::mean_dim(nll(logits, targets), 1), {s});
    }

    // src/nn/loss.rs:27-34: sum(nll · mask) / max(count, 1)
    static Tensor masked_cross_entropy(const Tensor& logits, const Int& targets, const Tensor& mask) {
        size_t s = logits.sh[0], n = logits.sh[1] * logits.sh[2];
        Tensor l = nll(logits, targets);
        Tensor m = E::reshape(mask, {s, n});
        Tensor count = E::reshape(E::clamp_min(E::sum_dim(m, 1), 1.0), {s});
        return E::div(E::reshape(E::sum_dim(E::mul(l, m), 1), {s}), count);
    }

    // src/nn/loss.rs:48-79
    static Tensor cross_entropy_with(const Tensor& logits, const Int& targets, const Tensor* mask, const CeOptions& o) {
        if (o.is_default()) return mask ? masked_cross_entropy(logits, targets, *mask) : cross_entropy(logits, targets);
        if (!(o.smoothing >= 0.0 && o.smoothing <= 1.0)) fail("label smoothing outside [0, 1]");
        size_t s = logits.sh[0], n = logits.sh[1] * logits.sh[2], v = logits.sh[3];
        std::vector<double> keep(s * n, 1.0);
        if (mask)
            for (size_t i = 0; i < s * n; i++) keep[i] = (double)mask->v()[i];
        std::vector<int64_t> tv = targets.v;
        for (size_t i = 0; i < s * n; i++)
            if (o.has_ignore_index && tv[i] == o.ignore_index) {  // ignored targets read class 0
                keep[i] = 0.0;
                tv[i] = 0;
            }
        Tensor logp = E::reshape(E::log_softmax(logits, 3), {s, n, v});
        Tensor onehot = E::one_hot(Int{tv, Shape{s, n}}, v);
        Tensor l = E::neg(E::reshape(E::sum_dim(E::mul(logp, onehot), 2), {s, n}));
        if (o.smoothing > 0.0) {
            Tensor uniform = E::neg(E::reshape(E::mean_dim(logp, 2), {s, n}));
            l = E::add(E::mul_scalar(l, 1.0 - o.smoothing), E::mul_scalar(uniform, o.smoothing));
        }
        Tensor k = Tensor::from_f64s(keep.data(), Shape{s, n});
        Tensor count = E::reshape(E::clamp_min(E::sum_dim(k, 1), 1.0), {s});
        return E::div(E::reshape(E::sum_dim(E::mul(l, k), 1), {s}), count);
    }

    // src/nn/loss.rs:175-183: per-seed mean over positions of KL(softmax(target) ‖ softmax(pred))
    static Tensor kl_div(const Tensor& pred_logits, const Tensor& target_logits) {
        size_t r = pred_logits.rank(), s = pred_logits.sh[0];
        size_t n = pred_logits.n() / s / pred_logits.sh[r - 1];
        Tensor logq = E::log_softmax(pred_logits, r - 1);
        Tensor logp = E::log_softmax(target_logits, r - 1);
        Tensor per = E::sum_dim(E::mul(E::exp(logp), E::sub(logp, logq)), r - 1);
        return E::reshape(E::mean_dim(E::reshape(per, {s, n}), 1), {s});
    }
};

}  // namespace orc
