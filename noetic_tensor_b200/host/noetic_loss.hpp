// noetic::nn::loss — the cross-entropy family over libnrl.so, in C++ (src/nn/loss.rs:10-79,
// 175-183): the same names, per-seed results [S], options and error texts as the reference, on
// the tensors and tape of noetic_rl.hpp. One tape node per call.
#pragma once
#include "noetic_rl.hpp"

namespace noetic {
namespace nn {
namespace loss {

// src/nn/loss.rs:36-43
struct CeOptions {
    bool has_ignore_index = false;
    int64_t ignore_index = 0;
    double smoothing = 0.0;
    static CeOptions ignore(int64_t i) { CeOptions o; o.has_ignore_index = true; o.ignore_index = i; return o; }
    CeOptions with_smoothing(double e) const { CeOptions o = *this; o.smoothing = e; return o; }
    bool is_default() const { return !has_ignore_index && smoothing == 0.0; }
};

namespace detail {
using rl::detail::Saved;
using rl::detail::stream;

// targets → device I32 and the not-ignored weights; ignored targets read class 0 (loss.rs:60-65)
inline void check_targets(std::vector<int64_t>& t, size_t V, const CeOptions& o, std::vector<float>* keep) {
    for (size_t i = 0; i < t.size(); i++) {
        if (o.has_ignore_index && t[i] == o.ignore_index) {
            (*keep)[i] = 0.f;
            t[i] = 0;
        }
        if (t[i] < 0 || (uint64_t)t[i] >= V) throw std::runtime_error("one_hot: " + std::to_string(t[i]) + " is outside 0.." + std::to_string(V));
    }
}

// the shared body: per-position loss, optional per-seed mean, one tape node
inline Tensor ce(const Tensor& logits, const IntTensor& targets, const Tensor* mask, const CeOptions& o, bool reduce) {
    if (logits.rank() != 4) throw std::runtime_error("logits [S, B, T, V]");
    const size_t S = logits.shape()[0], N = logits.shape()[1] * logits.shape()[2], V = logits.shape()[3], n = S * N;
    if (targets.data.size() != n) throw std::runtime_error("targets [S, B, T]");
    if (mask && numel(mask->shape()) != n) throw std::runtime_error("mask [S, B, T]");
    std::vector<int64_t> t = targets.data;
    std::vector<float> keep_h;
    bool has_keep = mask != nullptr || o.has_ignore_index;
    if (has_keep) keep_h = mask ? mask->reshape(Shape{n}).to_vec() : std::vector<float>(n, 1.f);
    check_targets(t, V, o, has_keep ? &keep_h : nullptr);
    Device dev = logits.device();
    auto s = std::make_shared<Saved>();
    auto logp = std::make_shared<Tensor>(Tensor::empty(Shape{n}, DType::F32, dev));
    // token_log_probs of the (rewritten) targets
    IntTensor tt = IntTensor::from_data(t, rl::detail::lead(logits));
    rl::detail::forward(logits, nullptr, &tt, *s, logp.get(), false, false);
    std::shared_ptr<Tensor> keep, zsum;
    if (has_keep) keep = std::make_shared<Tensor>(Tensor::from_f32(keep_h, Shape{n}, dev));
    if (o.smoothing > 0.0) {
        zsum = std::make_shared<Tensor>(Tensor::empty(Shape{n}, DType::F32, dev));
        nrl(nrl_row_sum(rl::detail::dt(logits), n, (uint32_t)V, logits.dev(), zsum->dev(), stream()), "row_sum");
    }
    auto args = std::make_shared<nrl_ce_args>();
    std::memset(args.get(), 0, sizeof(nrl_ce_args));
    args->struct_size = sizeof(nrl_ce_args);
    args->V = (uint32_t)V;
    args->n = n;
    args->smoothing = o.smoothing;
    args->logp = logp->dev();
    args->rowstats = s->rowstats.dev();
    args->logit_sum = zsum ? zsum->dev() : 0;
    args->keep = keep ? keep->dev() : 0;
    Tensor per = Tensor::empty(Shape{S, 1, N}, DType::F32, dev);
    nrl_ce_args fa = *args;
    fa.loss = per.dev();
    nrl(nrl_ce_tokens(&fa, stream()), "ce_tokens");
    Tensor out;
    if (reduce) {
        out = Tensor::empty(Shape{S}, DType::F32, dev);
        nrl(nrl_reduce_tokens(NRL_REDUCE_TOKEN_MEAN, S, 1, N, per.dev(), keep ? keep->dev() : 0, out.dev(), stream()), "reduce_tokens");
    } else {
        out = per.reshape(Shape{S, N});
    }
    if (logits.tracked()) {
        Tensor leaf = logits;
        out.node_ = std::make_shared<Node>();
        out.node_->id = Tensor::next_id();
        out.node_->parents = {logits.node_};
        out.node_->backward = [=](const Tensor& g, std::map<uint64_t, Tensor>& grads) {
            Tensor d_per = g;
            if (reduce) {
                d_per = Tensor::empty(Shape{n}, DType::F32, dev);
                nrl(nrl_reduce_tokens_bwd(NRL_REDUCE_TOKEN_MEAN, S, 1, N, keep ? keep->dev() : 0, g.dev(), d_per.dev(), stream()), "reduce_tokens_bwd");
            }
            Tensor g_lp = Tensor::empty(Shape{n}, DType::F32, dev), g_un;
            nrl_ce_args ba = *args;
            ba.upstream = d_per.dev();
            ba.g_logp = g_lp.dev();
            if (o.smoothing > 0.0) {
                g_un = Tensor::empty(Shape{n}, DType::F32, dev);
                ba.g_uniform = g_un.dev();
            }
            nrl(nrl_ce_tokens(&ba, stream()), "ce_tokens backward");
            rl::detail::push_logits_grad(*s, leaf, &g_lp, nullptr, nullptr, grads, o.smoothing > 0.0 ? &g_un : nullptr);
            (void)logp;
            (void)zsum;
        };
    }
    return out;
}
}  // namespace detail

// src/nn/loss.rs:10-16 → [S, B·T]
inline Tensor nll(const Tensor& logits, const IntTensor& targets) { return detail::ce(logits, targets, nullptr, CeOptions(), false); }
// src/nn/loss.rs:19-22 → [S]
inline Tensor cross_entropy(const Tensor& logits, const IntTensor& targets) { return detail::ce(logits, targets, nullptr, CeOptions(), true); }
// src/nn/loss.rs:27-34 → [S]
inline Tensor masked_cross_entropy(const Tensor& logits, const IntTensor& targets, const Tensor& mask) { return detail::ce(logits, targets, &mask, CeOptions(), true); }
// src/nn/loss.rs:48-79 → [S]
inline Tensor cross_entropy_with(const Tensor& logits, const IntTensor& targets, const Tensor* mask, const CeOptions& opts) {
    if (!opts.is_default() && !(opts.smoothing >= 0.0 && opts.smoothing <= 1.0)) throw std::runtime_error("label smoothing " + std::to_string(opts.smoothing) + " outside [0, 1]");
    return detail::ce(logits, targets, mask, opts, true);
}

// src/nn/loss.rs:175-183: per-seed mean over positions of KL(softmax(target) ‖ softmax(pred));
// gradients flow to whichever side is tracked.
inline Tensor kl_div(const Tensor& pred_logits, const Tensor& target_logits) {
    if (pred_logits.shape() != target_logits.shape() || pred_logits.dtype() != target_logits.dtype()) throw std::runtime_error("kl_div: shapes differ");
    const size_t S = pred_logits.shape()[0], V = pred_logits.shape().back(), n = numel(pred_logits.shape()) / V, N = n / S;
    Device dev = pred_logits.device();
    auto s = std::make_shared<rl::detail::Saved>();
    rl::detail::forward(target_logits, &pred_logits, nullptr, *s, nullptr, true, false);  // policy side = the target
    Tensor out = Tensor::empty(Shape{S}, DType::F32, dev);
    nrl(nrl_reduce_tokens(NRL_REDUCE_TOKEN_MEAN, S, 1, N, s->kl.dev(), 0, out.dev(), rl::detail::stream()), "reduce_tokens");
    if (pred_logits.tracked() || target_logits.tracked()) {
        Tensor q = pred_logits, p = target_logits;
        out.node_ = std::make_shared<Node>();
        out.node_->id = Tensor::next_id();
        if (q.tracked()) out.node_->parents.push_back(q.node_);
        if (p.tracked()) out.node_->parents.push_back(p.node_);
        out.node_->backward = [=](const Tensor& g, std::map<uint64_t, Tensor>& grads) {
            Tensor d_per = Tensor::empty(Shape{n}, DType::F32, dev);
            nrl(nrl_reduce_tokens_bwd(NRL_REDUCE_TOKEN_MEAN, S, 1, N, 0, g.dev(), d_per.dev(), rl::detail::stream()), "reduce_tokens_bwd");
            rl::detail::push_kl_grads(*s, p, q, d_per, grads);
        };
    }
    return out;
}

}  // namespace loss
}  // namespace nn
}  // namespace noetic
