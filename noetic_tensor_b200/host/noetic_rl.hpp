// noetic::nn::rl over libnrl.so — the host side of the drop-in, in C++.
//
// The reference crate is Rust; where no Rust toolchain is at hand this header is the host-side
// mirror of its `nn::rl` interface (src/nn/rl.rs): the same function names, argument meanings,
// reductions and error behaviour, on device-resident tensors, with a small tape so that
// `backward` yields d(logits) as the reference's `run_backward` does
// (src/tensor/autodiff.rs:141-215). Each rl function is ONE tape node calling the fused kernels
// of include/nrl.h, where the reference records ~40 generic nodes per PPO step.
//
// Scope: what `nn::rl` needs and nothing else — a contiguous device Tensor (F32 / BF16 logits,
// F32 per-token values, U8 masks), a host IntTensor of tokens (the reference's IntTensor is
// host-resident i64, src/tensor/int.rs:14-18), gradients with respect to logits tensors.
// Errors are C++ exceptions carrying the reference's messages where it panics.
#pragma once
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/nrl.h"

namespace noetic {

enum class DType { F32, BF16, U8, I32 };
inline size_t dtype_size(DType d) { return d == DType::F32 || d == DType::I32 ? 4 : (d == DType::BF16 ? 2 : 1); }

struct Device {
    int index;
    static Device Cuda(int i) { return Device{i}; }  // src/tensor/device.rs:22-27
};

inline void cu(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA ") + what + ": " + cudaGetErrorString(e));
}
inline void nrl(int rc, const char* what) {
    if (rc != 0) throw std::runtime_error(std::string("nrl ") + what + ": " + nrl_error_string(rc));
}

typedef std::vector<size_t> Shape;
inline size_t numel(const Shape& s) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    return n;
}

class Tensor;
struct Node {
    uint64_t id;
    std::vector<std::shared_ptr<Node>> parents;
    // receives this node's gradient; adds its parents' gradients into `grads`
    std::function<void(const Tensor& g, std::map<uint64_t, Tensor>& grads)> backward;
};

// bf16 round-to-nearest-even, as src/tensor/half.rs:15-27
inline uint16_t bf16_from_f32(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    if (x != x) return (uint16_t)((b >> 16) | 0x0040);
    return (uint16_t)((b + 0x7fff + ((b >> 16) & 1)) >> 16);
}

class Tensor {
public:
    Tensor() {}
    static Tensor empty(const Shape& shape, DType dt, Device dev) {
        Tensor t;
        t.shape_ = shape;
        t.dtype_ = dt;
        t.device_ = dev;
        cu(cudaSetDevice(dev.index), "set device");
        void* p = nullptr;
        size_t bytes = numel(shape) * dtype_size(dt);
        cu(cudaMalloc(&p, bytes ? bytes : 1), "alloc");
        t.buf_ = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
        return t;
    }
    static Tensor from_f32(const std::vector<float>& v, const Shape& shape, Device dev, DType dt = DType::F32) {
        if (v.size() != numel(shape)) throw std::runtime_error("tensor: data does not match shape");
        Tensor t = empty(shape, dt, dev);
        if (dt == DType::F32) {
            cu(cudaMemcpy(t.ptr(), v.data(), v.size() * 4, cudaMemcpyHostToDevice), "upload");
        } else if (dt == DType::BF16) {
            std::vector<uint16_t> h(v.size());
            for (size_t i = 0; i < v.size(); i++) h[i] = bf16_from_f32(v[i]);
            cu(cudaMemcpy(t.ptr(), h.data(), h.size() * 2, cudaMemcpyHostToDevice), "upload");
        } else {
            throw std::runtime_error("from_f32: float dtypes only");
        }
        return t;
    }
    static Tensor from_u8(const std::vector<uint8_t>& v, const Shape& shape, Device dev) {
        Tensor t = empty(shape, DType::U8, dev);
        cu(cudaMemcpy(t.ptr(), v.data(), v.size(), cudaMemcpyHostToDevice), "upload");
        return t;
    }
    std::vector<float> to_vec() const {
        if (dtype_ != DType::F32) throw std::runtime_error("to_vec: F32 only");
        std::vector<float> v(numel(shape_));
        cu(cudaMemcpy(v.data(), ptr(), v.size() * 4, cudaMemcpyDeviceToHost), "download");
        return v;
    }
    const Shape& shape() const { return shape_; }
    size_t rank() const { return shape_.size(); }
    DType dtype() const { return dtype_; }
    Device device() const { return device_; }
    void* ptr() const { return buf_.get(); }
    nrl_devptr dev() const { return (nrl_devptr)(uintptr_t)buf_.get(); }
    Tensor reshape(const Shape& s) const {
        if (numel(s) != numel(shape_)) throw std::runtime_error("reshape: element count");
        Tensor t = *this;
        t.shape_ = s;
        return t;
    }
    // a leaf whose gradient `backward` reports (src/tensor/float.rs require_grad)
    Tensor require_grad() const {
        Tensor t = detach();
        t.node_ = std::make_shared<Node>();
        t.node_->id = next_id();
        return t;
    }
    Tensor detach() const {
        Tensor t = *this;
        t.node_ = nullptr;
        return t;
    }
    bool tracked() const { return (bool)node_; }
    std::shared_ptr<Node> node_;
    static uint64_t next_id() {
        static uint64_t n = 0;
        return ++n;
    }

    // tempered_logits state: a lazy view (temperature and masks are applied inside the kernels)
    float tau_ = 1.0f;
    std::shared_ptr<Tensor> add_mask_, allow_mask_;

private:
    Shape shape_;
    DType dtype_ = DType::F32;
    Device device_{0};
    std::shared_ptr<void> buf_;
};

// Host-resident i64 tokens (src/tensor/int.rs:14-18)
struct IntTensor {
    std::vector<int64_t> data;
    Shape shape;
    static IntTensor from_data(std::vector<int64_t> v, Shape s) { return IntTensor{std::move(v), std::move(s)}; }
};

struct Gradients {
    std::map<uint64_t, Tensor> map;
    const Tensor* grad(const Tensor& t) const {
        if (!t.node_) return nullptr;
        auto it = map.find(t.node_->id);
        return it == map.end() ? nullptr : &it->second;
    }
};

// One term of a total loss: Σ value·weight (weight 1 per element when `scale` alone is given).
struct Term {
    Tensor value;
    double scale = 1.0;
};

// backward of Σ_k scale_k · value_k.sum(): what `(a + b * β − c * h).backward()` is in the
// reference, for rl values a, b, h. Nodes run in reverse creation order, so the gradients of a
// logits tensor that several terms use are summed in a fixed order.
inline Gradients backward(const std::vector<Term>& terms) {
    Gradients out;
    std::map<uint64_t, std::shared_ptr<Node>, std::greater<uint64_t>> todo;
    std::function<void(const std::shared_ptr<Node>&)> collect = [&](const std::shared_ptr<Node>& n) {
        if (todo.count(n->id)) return;
        todo[n->id] = n;
        for (auto& p : n->parents) collect(p);
    };
    std::map<uint64_t, Tensor> grads;
    for (const Term& t : terms) {
        if (!t.value.node_) throw std::runtime_error("backward on an untracked tensor");
        if (grads.count(t.value.node_->id)) throw std::runtime_error("backward: a value listed twice");
        collect(t.value.node_);
        grads[t.value.node_->id] = Tensor::from_f32(std::vector<float>(numel(t.value.shape()), (float)t.scale), t.value.shape(), t.value.device());
    }
    for (auto& kv : todo) {
        auto it = grads.find(kv.first);
        if (it == grads.end() || !kv.second->backward) continue;  // a leaf keeps its gradient
        Tensor g = it->second;
        grads.erase(it);
        kv.second->backward(g, grads);
    }
    out.map = std::move(grads);
    return out;
}
inline Gradients backward(const Tensor& value) { return backward(std::vector<Term>{Term{value, 1.0}}); }
// (value * upstream).sum().backward(), upstream of the value's shape
inline Gradients backward(const Tensor& value, const Tensor& upstream) {
    if (!value.node_) throw std::runtime_error("backward on an untracked tensor");
    if (numel(upstream.shape()) != numel(value.shape())) throw std::runtime_error("backward: upstream shape");
    Gradients out;
    std::map<uint64_t, std::shared_ptr<Node>, std::greater<uint64_t>> todo;
    std::function<void(const std::shared_ptr<Node>&)> collect = [&](const std::shared_ptr<Node>& n) {
        if (todo.count(n->id)) return;
        todo[n->id] = n;
        for (auto& p : n->parents) collect(p);
    };
    collect(value.node_);
    std::map<uint64_t, Tensor> grads;
    grads[value.node_->id] = upstream.reshape(value.shape());
    for (auto& kv : todo) {
        auto it = grads.find(kv.first);
        if (it == grads.end() || !kv.second->backward) continue;
        Tensor g = it->second;
        grads.erase(it);
        kv.second->backward(g, grads);
    }
    out.map = std::move(grads);
    return out;
}

namespace nn {
namespace rl {

// src/nn/rl.rs:36-55
enum class TokenReduction { None = 0, Sum = 1, TokenMean = 2, PerSequence = 3, SequenceMean = 4 };
// src/nn/rl.rs:356-364
enum class KlEstimator { K1 = NRL_LOSS_K1, K2 = NRL_LOSS_K2, K3 = NRL_LOSS_K3 };
constexpr double LOG_RATIO_CLAMP = 20.0;  // src/nn/rl.rs:146
constexpr double KL_DELTA_CLAMP = 20.0;   // src/nn/rl.rs:150

// src/nn/rl.rs:160-198
struct Clip {
    double low, high;
    bool has_dual = false;
    double dual = 0.0;
    bool has_log_ratio_clamp = true;
    double log_ratio_clamp = LOG_RATIO_CLAMP;
    static Clip make(double low, double high) { return Clip{low, high}; }
    static Clip symmetric(double eps) { return Clip{eps, eps}; }
    Clip with_dual(double c) const { Clip k = *this; k.has_dual = true; k.dual = c; return k; }
    Clip with_log_ratio_clamp(bool on, double b = LOG_RATIO_CLAMP) const { Clip k = *this; k.has_log_ratio_clamp = on; k.log_ratio_clamp = b; return k; }
    void check() const {
        if (!(low >= 0.0 && low < 1.0 && high >= 0.0 && std::isfinite(low) && std::isfinite(high))) throw std::runtime_error("clip range (need 0 <= low < 1, 0 <= high)");
        if (has_dual && !(dual > 1.0 && std::isfinite(dual))) throw std::runtime_error("dual clip (need c > 1)");
        if (has_log_ratio_clamp && !(log_ratio_clamp > 0.0)) throw std::runtime_error("log-ratio clamp (need b > 0)");
    }
};

namespace detail {
inline cudaStream_t stream() { return 0; }
inline uint32_t dt(const Tensor& t) {
    if (t.dtype() == DType::F32) return NRL_F32;
    if (t.dtype() == DType::BF16) return NRL_BF16;
    throw std::runtime_error("logits must be F32 or BF16");
}
struct Rows {
    uint64_t rows;
    uint32_t V;
};
inline Rows rows_of(const Tensor& logits) {
    if (logits.rank() < 1) throw std::runtime_error("logits of rank 0");
    uint32_t V = (uint32_t)logits.shape().back();
    return Rows{numel(logits.shape()) / V, V};
}
inline Shape lead(const Tensor& logits) { return Shape(logits.shape().begin(), logits.shape().end() - 1); }
inline void fill_inputs(nrl_row_fwd_args& a, const Tensor& z, const Tensor* ref) {
    Rows r = rows_of(z);
    std::memset(&a, 0, sizeof a);
    a.struct_size = sizeof a;
    a.dtype = dt(z);
    a.V = r.V;
    a.rows = r.rows;
    a.temperature = z.tau_;
    a.logits = z.dev();
    if (ref) {
        if (ref->shape() != z.shape() || ref->dtype() != z.dtype()) throw std::runtime_error("categorical_kl: reference logits shape");
        a.ref_logits = ref->dev();
    }
    if (z.allow_mask_ && z.allow_mask_->dtype() == DType::I32) {
        // bit-packed: I32 words [..., ceil(V/32)] (or one row), bit v of a row = bit v mod 32 of word v / 32
        const size_t words = z.allow_mask_->shape().back();
        a.allow_mask = z.allow_mask_->dev();
        a.allow_row_stride = numel(z.allow_mask_->shape()) == words && r.rows != 1 ? 0 : words;
        a.flags |= NRL_FWD_MASK_BITS;
    } else if (z.allow_mask_) {
        a.allow_mask = z.allow_mask_->dev();
        a.allow_row_stride = numel(z.allow_mask_->shape()) == r.V && r.rows != 1 ? 0 : r.V;
    }
    if (z.add_mask_) {
        a.add_mask = z.add_mask_->dev();
        a.add_row_stride = numel(z.add_mask_->shape()) == r.V && r.rows != 1 ? 0 : r.V;
    }
}
struct Saved {  // what one forward leaves for its backward (O(rows), not the [rows, V] log-softmax)
    Tensor z, ref, tokens, rowstats, kl, entropy;
    bool has_ref = false;
};
inline void row_bwd(const Saved& s, const Tensor* g_lp, const Tensor* g_kl, const Tensor* g_en, Tensor* d, bool accumulate, const Tensor* g_un = nullptr, Tensor* d_ref = nullptr) {
    nrl_row_fwd_args f;
    fill_inputs(f, s.z, s.has_ref ? &s.ref : nullptr);
    nrl_row_bwd_args b;
    std::memset(&b, 0, sizeof b);
    b.struct_size = sizeof b;
    b.dtype = f.dtype; b.V = f.V; b.temperature = f.temperature; b.rows = f.rows;
    b.logits = f.logits; b.ref_logits = f.ref_logits; b.allow_mask = f.allow_mask; b.allow_row_stride = f.allow_row_stride;
    b.add_mask = f.add_mask; b.add_row_stride = f.add_row_stride;
    b.mask_bits = (f.flags & NRL_FWD_MASK_BITS) ? 1 : 0;
    b.tokens = g_lp ? s.tokens.dev() : 0;
    b.rowstats = s.rowstats.dev();
    b.kl = g_kl ? s.kl.dev() : 0;
    b.entropy = g_en ? s.entropy.dev() : 0;
    b.g_logp = g_lp ? g_lp->dev() : 0;
    b.g_kl = g_kl ? g_kl->dev() : 0;
    b.g_ent = g_en ? g_en->dev() : 0;
    b.g_uniform = g_un ? g_un->dev() : 0;
    b.d_logits = d ? d->dev() : 0;
    b.d_ref_logits = d_ref ? d_ref->dev() : 0;
    b.accumulate = accumulate ? 1 : 0;
    nrl(nrl_row_bwd(&b, stream()), "row_bwd");
}
// add this node's d(logits) into the gradient map (the tape's `new + old`)
inline void push_logits_grad(const Saved& s, const Tensor& logits_leaf, const Tensor* g_lp, const Tensor* g_kl, const Tensor* g_en, std::map<uint64_t, Tensor>& grads, const Tensor* g_un = nullptr) {
    auto it = grads.find(logits_leaf.node_->id);
    if (it == grads.end()) {
        Tensor d = Tensor::empty(logits_leaf.shape(), DType::F32, logits_leaf.device());
        row_bwd(s, g_lp, g_kl, g_en, &d, false, g_un);
        grads[logits_leaf.node_->id] = d;
    } else {
        row_bwd(s, g_lp, g_kl, g_en, &it->second, true, g_un);
    }
}
// the KL term's gradients to both sides: `policy` is the side the forward streamed as logits,
// `reference` the side it streamed as ref_logits; either may be untracked
inline void push_kl_grads(const Saved& s, const Tensor& policy, const Tensor& reference, const Tensor& g_kl, std::map<uint64_t, Tensor>& grads) {
    auto slot = [&](const Tensor& leaf, bool& fresh) -> Tensor {
        auto it = grads.find(leaf.node_->id);
        fresh = it == grads.end();
        return fresh ? Tensor::empty(leaf.shape(), DType::F32, leaf.device()) : it->second;
    };
    // one launch per side that already holds a gradient differently from the other; one for both otherwise
    bool fp = true, fr = true;
    Tensor dp, dr;
    if (policy.tracked()) dp = slot(policy, fp);
    if (reference.tracked()) dr = slot(reference, fr);
    if (policy.tracked() && reference.tracked() && fp != fr) {
        row_bwd(s, nullptr, &g_kl, nullptr, &dp, !fp);
        row_bwd(s, nullptr, &g_kl, nullptr, nullptr, !fr, nullptr, &dr);
    } else {
        row_bwd(s, nullptr, &g_kl, nullptr, policy.tracked() ? &dp : nullptr, policy.tracked() ? !fp : !fr, nullptr, reference.tracked() ? &dr : nullptr);
    }
    if (policy.tracked()) grads[policy.node_->id] = dp;
    if (reference.tracked()) grads[reference.node_->id] = dr;
}
inline Tensor zeros_like_rows(uint64_t n, Device dev, DType dt = DType::F32) { return Tensor::empty(Shape{(size_t)n}, dt, dev); }
inline Tensor reduce(const Tensor& per, const Tensor* mask, TokenReduction r) {
    const Shape& s = per.shape();
    if (s.size() != 3) throw std::runtime_error("per-token values [S, B, T]");
    Shape os = r == TokenReduction::None ? s : (r == TokenReduction::PerSequence ? Shape{s[0], s[1]} : Shape{s[0]});
    Tensor out = Tensor::empty(os, DType::F32, per.device());
    nrl(nrl_reduce_tokens((uint32_t)r, s[0], s[1], s[2], per.dev(), mask ? mask->dev() : 0, out.dev(), stream()), "reduce_tokens");
    return out;
}
inline Tensor reduce_bwd(const Shape& s, const Tensor* mask, TokenReduction r, const Tensor& g, Device dev) {
    Tensor d = Tensor::empty(s, DType::F32, dev);
    nrl(nrl_reduce_tokens_bwd((uint32_t)r, s[0], s[1], s[2], mask ? mask->dev() : 0, g.dev(), d.dev(), stream()), "reduce_tokens_bwd");
    return d;
}
inline void check_mask(const Tensor* mask, const Tensor& like) {
    if (mask && mask->shape() != like.shape()) throw std::runtime_error("rl: mask shape");
}
}  // namespace detail

// src/nn/rl.rs:475-486. The mask is additive F32 (−inf or −1e9 exclude) or a U8 allow-mask, of
// shape [..., V] broadcastable as [1, V] or [rows, V]. Nothing is materialised.
inline Tensor tempered_logits(const Tensor& logits, double temperature, const Tensor* mask) {
    if (!(temperature > 0.0 && std::isfinite(temperature))) throw std::runtime_error("tempered_logits: temperature (must be positive)");
    Tensor z = logits;
    z.tau_ = (float)temperature * logits.tau_;
    if (mask) {
        const bool bits = mask->dtype() == DType::I32;  // a bit per token instead of a byte: I32 words [..., ceil(V/32)]
        if (bits ? mask->shape().back() != (logits.shape().back() + 31) / 32 : mask->shape().back() != logits.shape().back())
            throw std::runtime_error("tempered_logits: mask does not broadcast to the logits");
        if (mask->dtype() == DType::U8 || bits) z.allow_mask_ = std::make_shared<Tensor>(*mask);
        else if (mask->dtype() == DType::F32) z.add_mask_ = std::make_shared<Tensor>(*mask);
        else throw std::runtime_error("tempered_logits: mask dtype");
    }
    return z;
}

// src/nn/rl.rs:510-529, with the inverse-CDF sampler: one uniform in [0,1) per position
// (F32 [...]); temperature 0 is the first maximum and needs no uniforms.
inline IntTensor sample_categorical(const Tensor& logits, double temperature, const Tensor* mask, const Tensor* uniforms) {
    if (!(temperature >= 0.0 && std::isfinite(temperature))) throw std::runtime_error("sample_categorical: temperature (must be >= 0)");
    Tensor z = tempered_logits(logits.detach(), temperature == 0.0 ? 1.0 : temperature, mask);
    detail::Rows r = detail::rows_of(z);
    Tensor tok = Tensor::empty(Shape{(size_t)r.rows}, DType::I32, z.device());
    Tensor status = Tensor::empty(Shape{(size_t)r.rows}, DType::U8, z.device());
    Tensor ws;
    nrl_row_fwd_args a;
    detail::fill_inputs(a, z, nullptr);
    if (temperature == 0.0) {
        a.flags |= NRL_FWD_GREEDY;
    } else {
        if (!uniforms || numel(uniforms->shape()) != r.rows) throw std::runtime_error("sample_categorical: one uniform per position");
        a.flags |= NRL_FWD_SAMPLE;
        a.uniforms = uniforms->dev();
    }
    a.tokens = tok.dev();
    a.status = status.dev();
    uint64_t need = nrl_row_fwd_workspace_bytes(r.rows, r.V);
    if (need) {
        ws = Tensor::empty(Shape{(size_t)need}, DType::U8, z.device());
        a.workspace = ws.dev();
        a.workspace_bytes = need;
    }
    nrl(nrl_row_fwd(&a, detail::stream()), "row_fwd");
    uint64_t bad = 0;
    uint32_t bits = 0;
    int rc = nrl_check_status(status.dev(), r.rows, detail::stream(), &bad, &bits);
    if (rc == NRL_E_ROW_STATUS) throw std::runtime_error("sample_categorical: position " + std::to_string(bad) + " has no allowed token (every logit −∞ or a NaN)");
    nrl(rc, "check_status");
    std::vector<int32_t> h(r.rows);
    cu(cudaMemcpy(h.data(), tok.ptr(), h.size() * 4, cudaMemcpyDeviceToHost), "download tokens");
    IntTensor out;
    out.data.assign(h.begin(), h.end());
    out.shape = detail::lead(logits);
    return out;
}

// The state of a ChaCha20Rng (src/rng.rs:10-17 derives its 32-byte seed): the seed and the number
// of 32-bit words drawn so far.
struct ChaChaStream {
    uint8_t seed[32];
    uint64_t words = 0;
};

// src/nn/rl.rs:510-529 as the reference defines it: Gumbel-max with one `next_u64` of `rng` per
// logit in row-major order, so the tokens are the reference's for the same generator state;
// `rng` advances by what the reference's sampler draws. Temperature 0 draws nothing.
inline IntTensor sample_categorical(const Tensor& logits, double temperature, const Tensor* mask, ChaChaStream& rng) {
    if (!(temperature >= 0.0 && std::isfinite(temperature))) throw std::runtime_error("sample_categorical: temperature (must be >= 0)");
    if (temperature == 0.0) return sample_categorical(logits, 0.0, mask, (const Tensor*)nullptr);
    Tensor z = tempered_logits(logits.detach(), temperature, mask);
    detail::Rows r = detail::rows_of(z);
    Tensor tok = Tensor::empty(Shape{(size_t)r.rows}, DType::I32, z.device());
    Tensor status = Tensor::empty(Shape{(size_t)r.rows}, DType::U8, z.device());
    nrl_row_fwd_args f;
    detail::fill_inputs(f, z, nullptr);
    if (f.flags & NRL_FWD_MASK_BITS) throw std::runtime_error("sample_categorical with the reference's noise takes byte or additive masks, not bit-packed ones");
    nrl_gumbel_args a;
    std::memset(&a, 0, sizeof a);
    a.struct_size = sizeof a;
    a.dtype = f.dtype; a.V = f.V; a.temperature = f.temperature; a.rows = f.rows;
    a.logits = f.logits; a.allow_mask = f.allow_mask; a.allow_row_stride = f.allow_row_stride; a.add_mask = f.add_mask; a.add_row_stride = f.add_row_stride;
    std::memcpy(a.seed, rng.seed, 32);
    a.word_offset = rng.words;
    a.tokens = tok.dev();
    a.status = status.dev();
    nrl(nrl_sample_gumbel(&a, detail::stream()), "sample_gumbel");
    uint64_t bad = 0;
    uint32_t bits = 0;
    int rc = nrl_check_status(status.dev(), r.rows, detail::stream(), &bad, &bits);
    if (rc == NRL_E_ROW_STATUS) throw std::runtime_error("sample_categorical: position " + std::to_string(bad) + " has no allowed token (every logit −∞ or a NaN)");
    nrl(rc, "check_status");
    rng.words += 2ull * r.rows * r.V;
    std::vector<int32_t> h(r.rows);
    cu(cudaMemcpy(h.data(), tok.ptr(), h.size() * 4, cudaMemcpyDeviceToHost), "download tokens");
    IntTensor out;
    out.data.assign(h.begin(), h.end());
    out.shape = detail::lead(logits);
    return out;
}

namespace detail {
// One forward over the rows with given tokens and/or a reference; fills `s`.
inline void forward(const Tensor& z, const Tensor* ref, const IntTensor* tokens, Saved& s, Tensor* logp, bool want_kl, bool want_ent) {
    Rows r = rows_of(z);
    nrl_row_fwd_args a;
    fill_inputs(a, z, ref);
    s.z = z.detach();
    s.z.tau_ = z.tau_;
    s.z.add_mask_ = z.add_mask_;
    s.z.allow_mask_ = z.allow_mask_;
    s.has_ref = ref != nullptr;
    if (ref) s.ref = ref->detach();
    s.rowstats = Tensor::empty(Shape{(size_t)r.rows, 4}, DType::F32, z.device());
    a.rowstats = s.rowstats.dev();
    if (tokens) {
        if (tokens->shape != lead(z)) throw std::runtime_error("token_log_probs: tokens shape (the logits' without the vocabulary axis)");
        std::vector<int32_t> h(tokens->data.begin(), tokens->data.end());
        for (int64_t t : tokens->data)
            if (t < 0 || (uint64_t)t >= r.V) throw std::runtime_error("gather index out of range");
        s.tokens = Tensor::empty(Shape{(size_t)r.rows}, DType::I32, z.device());
        cu(cudaMemcpy(s.tokens.ptr(), h.data(), h.size() * 4, cudaMemcpyHostToDevice), "upload tokens");
        a.flags |= NRL_FWD_TOKENS_IN;
        a.tokens = s.tokens.dev();
        a.logp = logp->dev();
    }
    if (want_kl) {
        s.kl = Tensor::empty(Shape{(size_t)r.rows}, DType::F32, z.device());
        a.kl = s.kl.dev();
    }
    if (want_ent) {
        s.entropy = Tensor::empty(Shape{(size_t)r.rows}, DType::F32, z.device());
        a.entropy = s.entropy.dev();
    }
    Tensor ws;
    uint64_t need = nrl_row_fwd_workspace_bytes(r.rows, r.V);
    if (need) {
        ws = Tensor::empty(Shape{(size_t)need}, DType::U8, z.device());
        a.workspace = ws.dev();
        a.workspace_bytes = need;
    }
    nrl(nrl_row_fwd(&a, stream()), "row_fwd");
    cu(cudaStreamSynchronize(stream()), "sync");  // the workspace goes out of scope here
}
}  // namespace detail

// src/nn/rl.rs:134-141: log_softmax(logits)[…, tokens]; gradient onehot − softmax.
inline Tensor token_log_probs(const Tensor& logits, const IntTensor& tokens) {
    auto s = std::make_shared<detail::Saved>();
    Tensor logp = Tensor::empty(detail::lead(logits), DType::F32, logits.device());
    detail::forward(logits, nullptr, &tokens, *s, &logp, false, false);
    if (logits.tracked()) {
        Tensor leaf = logits;
        logp.node_ = std::make_shared<Node>();
        logp.node_->id = Tensor::next_id();
        logp.node_->parents = {logits.node_};
        logp.node_->backward = [s, leaf](const Tensor& g, std::map<uint64_t, Tensor>& grads) {
            Tensor flat = g.reshape(Shape{numel(g.shape())});
            detail::push_logits_grad(*s, leaf, &flat, nullptr, nullptr, grads);
        };
    }
    return logp;
}

// `token_log_probs(head(x), tokens)` and `categorical_entropy(head(x))` per position without the
// [.., V] logits in between (src/nn/decoder.rs:270-279 followed by src/nn/rl.rs:134-141, 405-414):
// `hidden` BF16 [.., d], `weight` BF16 [d, V] (the Linear's [in, out] layout, src/nn/linear.rs:1-3),
// tokens [..]. Returns the log-probabilities [..] and, if asked, the per-position entropies.
// Untracked: the backward of the fused form (d hidden, d weight) is not built; needs a
// compute-capability-10 device (tcgen05). `round_bf16`: statistics of the logits rounded to bf16.
namespace detail {
// the allow-mask of a fused head call: U8 [.., V] or [1, V], or I32 words of one bit per token [.., W] or [1, W]
inline void head_mask(nrl_readout_args& a, const Tensor* vocab_mask, uint64_t rows, uint64_t V) {
    if (!vocab_mask) return;
    if (vocab_mask->dtype() == DType::I32) {
        const uint64_t words = vocab_mask->shape().back(), n = numel(vocab_mask->shape());
        if (words < (V + 31) / 32 || (n != words && n != rows * words)) throw std::runtime_error("rl: mask shape");
        a.allow_mask = vocab_mask->dev();
        a.allow_row_stride = n == words ? 0 : words;
        a.flags |= NRL_READOUT_MASK_BITS;
        return;
    }
    if (vocab_mask->dtype() != DType::U8) throw std::runtime_error("rl: a U8 allow-mask or I32 words of bits");
    const uint64_t n = numel(vocab_mask->shape());
    if (n != V && n != rows * V) throw std::runtime_error("rl: mask shape");
    a.allow_mask = vocab_mask->dev();
    a.allow_row_stride = n == V ? 0 : V;
}
}  // namespace detail

// `vocab_mask` / `temperature`: the logits are the tempered ones (src/nn/rl.rs:475-486), what a rollout drawn by
// head_sample_categorical under the same mask and temperature is scored with.
inline Tensor head_token_log_probs(const Tensor& hidden, const Tensor& weight, const IntTensor& tokens, Tensor* entropy = nullptr, bool round_bf16 = false, const Tensor* vocab_mask = nullptr,
                                   double temperature = 1.0) {
    if (!(temperature > 0.0 && std::isfinite(temperature))) throw std::runtime_error("tempered_logits: temperature must be > 0");
    if (hidden.dtype() != DType::BF16 || weight.dtype() != DType::BF16) throw std::runtime_error("head_token_log_probs: BF16 hidden states and weight");
    if (hidden.rank() < 1 || weight.rank() != 2 || weight.shape()[0] != hidden.shape().back()) throw std::runtime_error("head_token_log_probs: hidden [.., d], weight [d, V]");
    const Shape lead(hidden.shape().begin(), hidden.shape().end() - 1);
    if (tokens.shape != lead) throw std::runtime_error("token_log_probs: tokens shape (the logits' without the vocabulary axis)");
    const uint64_t d = weight.shape()[0], V = weight.shape()[1], rows = numel(lead);
    std::vector<int32_t> h(tokens.data.begin(), tokens.data.end());
    for (int64_t t : tokens.data)
        if (t < 0 || (uint64_t)t >= V) throw std::runtime_error("gather index out of range");
    Tensor tok = Tensor::empty(Shape{(size_t)rows}, DType::I32, hidden.device());
    cu(cudaMemcpy(tok.ptr(), h.data(), h.size() * 4, cudaMemcpyHostToDevice), "upload tokens");
    Tensor logp = Tensor::empty(lead, DType::F32, hidden.device());
    Tensor status = Tensor::empty(Shape{(size_t)rows}, DType::U8, hidden.device());
    const uint64_t need = nrl_readout_workspace_bytes(rows, (uint32_t)V, (uint32_t)d, 0u);
    Tensor ws = Tensor::empty(Shape{(size_t)need}, DType::U8, hidden.device());
    nrl_readout_args a;
    std::memset(&a, 0, sizeof a);
    a.struct_size = sizeof a;
    a.flags = round_bf16 ? NRL_READOUT_ROUND_BF16 : 0u;
    a.temperature = (float)temperature;
    detail::head_mask(a, vocab_mask, rows, V);
    a.V = (uint32_t)V; a.d = (uint32_t)d; a.rows = rows;
    a.hidden = hidden.dev(); a.weights = weight.dev(); a.tokens = tok.dev();
    a.logp = logp.dev(); a.status = status.dev();
    if (entropy) {
        *entropy = Tensor::empty(lead, DType::F32, hidden.device());
        a.entropy = entropy->dev();
    }
    a.workspace = ws.dev(); a.workspace_bytes = need;
    nrl(nrl_readout_fwd(&a, detail::stream()), "readout_fwd");
    cu(cudaStreamSynchronize(detail::stream()), "sync");  // the workspace goes out of scope here
    return logp;
}

// `sample_categorical(head(x), 1.0, mask, ·)` by inverse CDF against one uniform per position without
// the [.., V] logits in between (src/nn/decoder.rs:270-279 followed by src/nn/rl.rs:490-529 with the
// path's sampler): `hidden` BF16 [.., d], `weight` BF16 [d, V], `uniforms` F32 [..] in [0, 1),
// `vocab_mask` an optional U8 allow-mask [.., V] or [1, V]. Returns the tokens (on the host, as
// sample_categorical does) and, if asked, their log-probabilities and the per-position entropies.
// Refuses a position with no allowed token with the reference's message (src/nn/rl.rs:516-519).
// `temperature` > 0 divides the logits (tempered_logits); 0 takes the first maximum (`uniforms` is not read then).
inline IntTensor head_sample_categorical(const Tensor& hidden, const Tensor& weight, const Tensor& uniforms, const Tensor* vocab_mask = nullptr, Tensor* logp = nullptr,
                                         Tensor* entropy = nullptr, double temperature = 1.0) {
    if (!(temperature >= 0.0 && std::isfinite(temperature))) throw std::runtime_error("sample_categorical: temperature (must be >= 0)");
    const bool greedy = temperature == 0.0;
    if (hidden.dtype() != DType::BF16 || weight.dtype() != DType::BF16) throw std::runtime_error("head_sample_categorical: BF16 hidden states and weight");
    if (hidden.rank() < 1 || weight.rank() != 2 || weight.shape()[0] != hidden.shape().back()) throw std::runtime_error("head_sample_categorical: hidden [.., d], weight [d, V]");
    const Shape lead(hidden.shape().begin(), hidden.shape().end() - 1);
    const uint64_t d = weight.shape()[0], V = weight.shape()[1], rows = numel(lead);
    if (!greedy && (uniforms.dtype() != DType::F32 || numel(uniforms.shape()) != rows)) throw std::runtime_error("sample_categorical: one uniform per position");
    nrl_readout_args a;
    std::memset(&a, 0, sizeof a);
    a.struct_size = sizeof a;
    a.flags = greedy ? NRL_READOUT_GREEDY : NRL_READOUT_SAMPLE;
    detail::head_mask(a, vocab_mask, rows, V);
    Tensor tok = Tensor::empty(Shape{(size_t)rows}, DType::I32, hidden.device());
    Tensor lp = Tensor::empty(lead, DType::F32, hidden.device());
    Tensor status = Tensor::empty(Shape{(size_t)rows}, DType::U8, hidden.device());
    const uint64_t need = nrl_readout_workspace_bytes(rows, (uint32_t)V, (uint32_t)d, a.flags);
    Tensor ws = Tensor::empty(Shape{(size_t)need}, DType::U8, hidden.device());
    a.V = (uint32_t)V; a.d = (uint32_t)d; a.rows = rows;
    a.hidden = hidden.dev(); a.weights = weight.dev(); a.tokens = tok.dev();
    if (!greedy) {
        a.uniforms = uniforms.dev();
        a.temperature = (float)temperature;
    }
    a.logp = lp.dev(); a.status = status.dev();
    if (entropy) {
        *entropy = Tensor::empty(lead, DType::F32, hidden.device());
        a.entropy = entropy->dev();
    }
    a.workspace = ws.dev(); a.workspace_bytes = need;
    nrl(nrl_readout_fwd(&a, detail::stream()), "readout_fwd");
    uint64_t bad = 0;
    uint32_t bits = 0;
    const int rc = nrl_check_status(status.dev(), rows, detail::stream(), &bad, &bits);  // a host read: the stream has drained
    if (rc == NRL_E_ROW_STATUS) throw std::runtime_error("sample_categorical: position " + std::to_string(bad) + " has no allowed token (every logit −∞ or a NaN)");
    nrl(rc, "check_status");
    std::vector<int32_t> h(rows);
    cu(cudaMemcpy(h.data(), tok.ptr(), h.size() * 4, cudaMemcpyDeviceToHost), "download tokens");
    if (logp) *logp = lp;
    IntTensor out;
    out.data.assign(h.begin(), h.end());
    out.shape = lead;
    return out;
}

// src/nn/rl.rs:204-211: every scored log-probability (mask != 0; no mask: all) is finite. Returns
// an empty string, or the reference's error text naming the first flat position. A host read.
inline std::string check_scored_finite(const std::string& what, const Tensor& logp, const Tensor* mask) {
    if (logp.dtype() != DType::F32) throw std::runtime_error("check_scored_finite: F32 log-probabilities");
    if (mask && numel(mask->shape()) != numel(logp.shape())) throw std::runtime_error("rl: mask shape");
    Tensor result = Tensor::empty(Shape{4}, DType::F32, logp.device());  // 16 bytes of device scratch
    uint64_t pos = 0;
    float value = 0.f;
    const int rc = nrl_check_scored_finite(logp.dev(), mask ? mask->dev() : 0, numel(logp.shape()), result.dev(), detail::stream(), &pos, &value);
    if (rc == NRL_E_NOT_FINITE) {
        const char* v = value != value ? "NaN" : (value > 0 ? "inf" : "-inf");  // Rust's `{}` of an f64
        return what + ": the scored log-probability at flat position " + std::to_string(pos) + " is " + v + " (not finite)";
    }
    nrl(rc, "check_scored_finite");
    return std::string();
}

// src/nn/rl.rs:213-221: the losses run the check in debug builds (here: unless NDEBUG is defined).
inline void debug_check(const char* what, const Tensor& logp, const Tensor* mask) {
#ifndef NDEBUG
    const std::string e = check_scored_finite(what, logp, mask);
    if (!e.empty()) throw std::runtime_error(e);
#else
    (void)what; (void)logp; (void)mask;
#endif
}

namespace detail {
// a token-level loss of logp [S,B,T]: one node whose backward hands d/dlogp to logp's node
inline Tensor token_level(uint32_t kind, const Tensor& logp, const Tensor* other, const Tensor* weights, const Tensor* mask, TokenReduction red, const Clip* clip, bool has_clamp, double clamp) {
    if (logp.rank() != 3) throw std::runtime_error("logp [S, B, T]");
    check_mask(mask, logp);
    const Shape s = logp.shape();
    auto args = std::make_shared<nrl_token_loss_args>();
    std::memset(args.get(), 0, sizeof(nrl_token_loss_args));
    args->struct_size = sizeof(nrl_token_loss_args);
    args->kind = kind;
    args->S = s[0]; args->B = s[1]; args->T = s[2];
    args->logp = logp.dev();
    if (other) {
        if (other->shape() != s) throw std::runtime_error("rl: old / reference log-probabilities shape");
        args->other = other->dev();
    }
    if (weights) {
        if (weights->rank() == 2) {
            if (weights->shape() != Shape{s[0], s[1]}) throw std::runtime_error("per-sequence weights [S, B]");
            args->weights_per_sequence = 1;
        } else if (weights->shape() != s) {
            throw std::runtime_error("per-token weights [S, B, T]");
        }
        args->weights = weights->dev();
    }
    if (mask) args->mask = mask->dev();
    if (clip) {
        clip->check();
        args->clip_low = clip->low; args->clip_high = clip->high;
        args->has_dual = clip->has_dual; args->dual = clip->dual;
        args->has_clamp = clip->has_log_ratio_clamp; args->clamp = clip->log_ratio_clamp;
    } else if (has_clamp) {
        if (!(clamp > 0.0)) throw std::runtime_error("kl_estimate: δ clamp (need b > 0)");
        args->has_clamp = 1; args->clamp = clamp;
    }
    Tensor per = Tensor::empty(s, DType::F32, logp.device());
    args->loss = per.dev();
    nrl(nrl_token_loss(args.get(), stream()), "token_loss");
    Tensor out = reduce(per, mask, red);
    if (logp.tracked()) {
        // keep the operands alive for the backward
        std::vector<Tensor> keep{logp.detach()};
        if (other) keep.push_back(*other);
        if (weights) keep.push_back(*weights);
        if (mask) keep.push_back(*mask);
        std::shared_ptr<Tensor> m = mask ? std::make_shared<Tensor>(*mask) : nullptr;
        Tensor lp = logp;
        out.node_ = std::make_shared<Node>();
        out.node_->id = Tensor::next_id();
        out.node_->parents = {logp.node_};
        out.node_->backward = [args, keep, m, red, s, lp](const Tensor& g, std::map<uint64_t, Tensor>& grads) {
            Tensor d_per = reduce_bwd(s, m.get(), red, g, lp.device());
            auto it = grads.find(lp.node_->id);  // a logp that feeds two losses: the second adds
            Tensor g_lp = it != grads.end() ? it->second : Tensor::empty(s, DType::F32, lp.device());
            nrl_token_loss_args a = *args;
            a.loss = 0;
            a.upstream = d_per.dev();
            a.dloss_dlogp = g_lp.dev();
            a.accumulate = it != grads.end();
            nrl(nrl_token_loss(&a, stream()), "token_loss backward");
            grads[lp.node_->id] = g_lp;
        };
    }
    return out;
}
}  // namespace detail

// src/nn/rl.rs:228-235
inline Tensor policy_gradient_loss(const Tensor& logp, const Tensor& weights, const Tensor* mask, TokenReduction reduction) {
    if (logp.rank() != 3) throw std::runtime_error("policy_gradient_loss: logp [S, B, T]");
    debug_check("policy_gradient_loss", logp, mask);
    return detail::token_level(NRL_LOSS_PG, logp, nullptr, &weights, mask, reduction, nullptr, false, 0.0);
}
// src/nn/rl.rs:265-287
inline Tensor clipped_policy_loss(const Tensor& logp, const Tensor& old_logp, const Tensor& advantages, const Tensor* mask, const Clip& clip, TokenReduction reduction) {
    clip.check();
    if (logp.rank() != 3) throw std::runtime_error("clipped_policy_loss: logp [S, B, T]");
    debug_check("clipped_policy_loss", logp, mask);
    debug_check("clipped_policy_loss (old log-probabilities)", old_logp, mask);
    return detail::token_level(NRL_LOSS_PPO, logp, &old_logp, &advantages, mask, reduction, &clip, false, 0.0);
}
// src/nn/rl.rs:380-400
inline Tensor kl_estimate(const Tensor& logp, const Tensor& ref_logp, KlEstimator e, bool has_delta_clamp, double delta_clamp, const Tensor* mask, TokenReduction reduction) {
    debug_check("kl_estimate", logp, mask);
    debug_check("kl_estimate (reference log-probabilities)", ref_logp, mask);
    return detail::token_level((uint32_t)e, logp, &ref_logp, nullptr, mask, reduction, nullptr, has_delta_clamp, delta_clamp);
}
// src/nn/rl.rs:293-317 (untracked)
inline Tensor clip_fraction(const Tensor& logp, const Tensor& old_logp, const Tensor& advantages, const Tensor* mask, const Clip& clip) {
    clip.check();
    const Shape s = logp.shape();
    nrl_token_loss_args a;
    std::memset(&a, 0, sizeof a);
    a.struct_size = sizeof a;
    a.kind = NRL_LOSS_PPO;
    a.S = s[0]; a.B = s[1]; a.T = s[2];
    a.logp = logp.dev(); a.other = old_logp.dev(); a.weights = advantages.dev();
    a.weights_per_sequence = advantages.rank() == 2;
    if (mask) a.mask = mask->dev();
    a.clip_low = clip.low; a.clip_high = clip.high; a.has_dual = clip.has_dual; a.dual = clip.dual;
    a.has_clamp = clip.has_log_ratio_clamp; a.clamp = clip.log_ratio_clamp;
    Tensor out = Tensor::empty(Shape{s[0]}, DType::F32, logp.device());
    nrl(nrl_clip_fraction(&a, out.dev(), detail::stream()), "clip_fraction");
    return out;
}

namespace detail {
inline Tensor row_level(bool kl, const Tensor& logits, const Tensor* ref, const Tensor* mask, TokenReduction red) {
    if (logits.rank() != 4) throw std::runtime_error(kl ? "categorical_kl: logits [S, B, T, V]" : "categorical_entropy: logits [S, B, T, V]");
    auto s = std::make_shared<Saved>();
    forward(logits, ref, nullptr, *s, nullptr, kl, !kl);
    Shape l = lead(logits);
    Tensor raw = (kl ? s->kl : s->entropy).reshape(l);
    if (mask) check_mask(mask, raw);
    Tensor per = raw;
    if (mask) {
        per = Tensor::empty(l, DType::F32, logits.device());
        nrl(nrl_mask_rows(numel(l), raw.dev(), mask->dev(), per.dev(), stream()), "mask_rows");
    }
    Tensor out = reduce(per, mask, red);
    if (logits.tracked()) {
        Tensor leaf = logits;
        std::shared_ptr<Tensor> m = mask ? std::make_shared<Tensor>(*mask) : nullptr;
        out.node_ = std::make_shared<Node>();
        out.node_->id = Tensor::next_id();
        out.node_->parents = {logits.node_};
        out.node_->backward = [s, leaf, m, red, l, kl](const Tensor& g, std::map<uint64_t, Tensor>& grads) {
            Tensor d_per = reduce_bwd(l, m.get(), red, g, leaf.device()).reshape(Shape{numel(l)});
            push_logits_grad(*s, leaf, nullptr, kl ? &d_per : nullptr, kl ? nullptr : &d_per, grads);
        };
    }
    return out;
}
}  // namespace detail

// src/nn/rl.rs:327-338
inline Tensor categorical_kl(const Tensor& logits, const Tensor& ref_logits, const Tensor* mask, TokenReduction reduction) {
    return detail::row_level(true, logits, &ref_logits, mask, reduction);
}
// src/nn/rl.rs:347-351: both sides at the sampling temperature under the same vocabulary mask
inline Tensor reference_kl(const Tensor& logits, const Tensor& ref_logits, double temperature, const Tensor* vocab_mask, const Tensor* mask, TokenReduction reduction) {
    return detail::row_level(true, tempered_logits(logits, temperature, vocab_mask), &ref_logits, mask, reduction);
}
// src/nn/rl.rs:405-414
inline Tensor categorical_entropy(const Tensor& logits, const Tensor* mask, TokenReduction reduction) {
    return detail::row_level(false, logits, nullptr, mask, reduction);
}

// src/nn/rl.rs:418-461: host f64, whatever the device
struct GroupNorm {
    bool std_norm = false;
    double eps = 0.0;
    bool unbiased = true;
    static GroupNorm MeanOnly() { return GroupNorm{}; }
    static GroupNorm Std(double eps, bool unbiased) { return GroupNorm{true, eps, unbiased}; }
};
inline std::vector<double> group_advantages(const std::vector<double>& rewards, size_t n, GroupNorm norm) {
    if (!(n >= 1 && rewards.size() % n == 0)) throw std::runtime_error("group_advantages: rewards in groups of n");
    if (norm.std_norm) {
        if (!(norm.eps >= 0.0)) throw std::runtime_error("group_advantages: ε < 0");
        if (norm.unbiased && n < 2) throw std::runtime_error("group_advantages: the sample standard deviation needs groups of at least 2");
    }
    std::vector<double> out;
    out.reserve(rewards.size());
    for (size_t g0 = 0; g0 < rewards.size(); g0 += n) {
        const double* g = rewards.data() + g0;
        double lo = INFINITY, hi = -INFINITY;
        for (size_t i = 0; i < n; i++) {
            lo = std::fmin(lo, g[i]);
            hi = std::fmax(hi, g[i]);
        }
        if (lo == hi) {
            out.insert(out.end(), n, 0.0);
            continue;
        }
        double sum = 0.0;
        for (size_t i = 0; i < n; i++) sum += g[i];
        const double mean = sum / (double)n;
        double scale = 1.0;
        if (norm.std_norm) {
            double ss = 0.0;
            for (size_t i = 0; i < n; i++) ss += (g[i] - mean) * (g[i] - mean);
            scale = std::sqrt(ss / (norm.unbiased ? (double)(n - 1) : (double)n)) + norm.eps;
        }
        for (size_t i = 0; i < n; i++) out.push_back((g[i] - mean) / scale);
    }
    return out;
}

// group_advantages_tensor (src/nn/rl.rs:465-469) over the last axis of device rewards [..., N],
// without the reference's host round trip: the same f64 operand order on the device, so the values
// are group_advantages' rounded to f32 once.
inline Tensor group_advantages_tensor(const Tensor& rewards, GroupNorm norm) {
    if (rewards.dtype() != DType::F32 || rewards.shape().empty()) throw std::runtime_error("group_advantages_tensor: F32 rewards of rank >= 1");
    const size_t n = rewards.shape().back();
    if (norm.std_norm) {
        if (!(norm.eps >= 0.0)) throw std::runtime_error("group_advantages: ε < 0");
        if (norm.unbiased && n < 2) throw std::runtime_error("group_advantages: the sample standard deviation needs groups of at least 2");
    }
    Tensor out = Tensor::empty(rewards.shape(), DType::F32, rewards.device());
    nrl(nrl_group_advantages(numel(rewards.shape()) / n, (uint32_t)n, norm.std_norm, norm.eps, norm.unbiased, rewards.dev(), out.dev(), detail::stream()), "group_advantages_tensor");
    return out;
}

}  // namespace rl
}  // namespace nn

// ---- lane operations of the tensor engine along the last axis (src/tensor/activation.rs:15-42,
// 71-77; Tensor::argmax / sum_dim on the last axis), forward values; untracked ------------------
namespace lane {
namespace detail {
inline Tensor run(uint32_t op, const Tensor& x, bool full, Tensor* index = nullptr) {
    if (x.shape().empty() || (x.dtype() != DType::F32 && x.dtype() != DType::BF16)) throw std::runtime_error("lane op: F32 or BF16 tensor of rank >= 1");
    const size_t V = x.shape().back();
    Shape os = x.shape();
    if (!full) os.back() = 1;
    Tensor out = Tensor::empty(os, DType::F32, x.device());
    nrl_lane_args a{};
    a.struct_size = sizeof(a);
    a.op = op;
    a.dtype = x.dtype() == DType::F32 ? NRL_F32 : NRL_BF16;
    a.V = (uint32_t)V;
    a.rows = numel(x.shape()) / V;
    a.x = x.dev();
    a.out = out.dev();
    if (index) {
        *index = Tensor::empty(os, DType::I32, x.device());
        a.out_index = index->dev();
    }
    nrl(nrl_lane_op(&a, 0), "lane op");
    return out;
}
}  // namespace detail
inline Tensor softmax(const Tensor& x) { return detail::run(NRL_LANE_SOFTMAX, x, true); }
inline Tensor log_softmax(const Tensor& x) { return detail::run(NRL_LANE_LOG_SOFTMAX, x, true); }
inline Tensor logsumexp(const Tensor& x) { return detail::run(NRL_LANE_LOGSUMEXP, x, false); }
inline Tensor sum_last(const Tensor& x) { return detail::run(NRL_LANE_SUM, x, false); }
// (index I32 [..., 1], value F32 [..., 1]): the first maximum, the first NaN of a lane that holds one
inline std::pair<Tensor, Tensor> argmax(const Tensor& x) {
    Tensor idx;
    Tensor val = detail::run(NRL_LANE_ARGMAX, x, false, &idx);
    return {idx, val};
}
}  // namespace lane
}  // namespace noetic
