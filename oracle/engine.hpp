// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of the slice of the noetic-tensor engine that `nn::rl` runs on: contiguous
// row-major float tensors, the element-wise / reduction / indexing kernels of the CPU backends
// and the reverse-mode tape. It exists only so that tests and the benchmark's CPU-baseline leg
// can check and time the reference's arithmetic; nothing shipped may include or link it.
//
// What it follows (paths inside the noetic-tensor repository):
//   src/tensor/kernels.rs:70-72    map
//   src/tensor/kernels.rs:108-118  zip with burn-style broadcasting (row-major output)
//   src/tensor/kernels.rs:122-148  unrolled_sum: eight partial sums, (p0+p4)+(p1+p5)+(p2+p6)+(p3+p7), tail
//   src/tensor/kernels.rs:153-174  sum_dim (last axis: unrolled_sum per lane; other axes: slices in order)
//   src/tensor/kernels.rs:184-209  argmax_dim: first maximum, NaN-propagating
//   src/tensor/kernels.rs:213-254  gather / scatter_add_zeros
//   src/tensor/backend.rs:63-72    Cpu(Fast) thresholds (map 2^20, zip 2^22, sums 2^22)
//   src/tensor/backend.rs:93-118   simd_sum: sixteen accumulators, then the remainder in order
//   src/tensor/backend.rs:143-239  Cpu(Fast): threaded map / same-shape zip / lane sums
//   src/tensor/float.rs:74-84      unbroadcast
//   src/tensor/float.rs:399-530    add/sub/mul/div, scalar ops, neg/exp/log/abs and their backward rules
//   src/tensor/float.rs:578-594    clamp_min / clamp_max / clamp as mask_fill of a comparison
//   src/tensor/float.rs:640-742    sum, sum_dim, max_dim, argmax
//   src/tensor/float.rs:984-1011   mask_fill, gather (backward: scatter_add into zeros)
//   src/tensor/autodiff.rs:78-127  record / attach: order = 1 + max input order, node iff an input is tracked
//   src/tensor/autodiff.rs:141-215 run_backward: burn's traversal, gradients summed `new + old`
//   src/tensor/activation.rs:30-42 log_softmax as one node, backward g − exp(y)·Σg
//
// Parity status: the Rust reference was not compiled for this build (no Rust toolchain), so this
// restatement is pinned against the hand-computed values and identities in the reference's own
// tests (src/nn/tests/rl.rs), restated in tests/test_oracle_golden.py. Rust's f32::exp / ln call
// the platform libm, as expf / logf do here; the build uses -ffp-contract=off and no fast-math
// because Rust neither contracts nor reassociates.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstddef>
#include <cstdlib>
#include <functional>
#include <limits>
#include <map>
#include <memory>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace orc {

enum class CpuMode { Reference, Fast };

struct Config {
    CpuMode mode = CpuMode::Reference;
    int threads = 1;  // NOETIC_THREADS of the Fast backend (src/tensor/backend.rs:58-61)
};
inline Config& config() {
    static Config c;
    return c;
}

typedef std::vector<size_t> Shape;

inline size_t numel(const Shape& s) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    return n;
}

[[noreturn]] inline void fail(const std::string& m) { throw std::runtime_error(m); }

// Thresholds of Cpu(Fast), src/tensor/backend.rs:63-72.
static const size_t FAST_MIN_MAP = size_t(1) << 20;
static const size_t FAST_MIN_ZIP = size_t(1) << 22;
static const size_t FAST_MIN_SUM = size_t(1) << 22;

// `fill` of src/tensor/backend.rs:76-91: n elements split into ceil(n/parts) chunks, one thread each.
template <class F>
inline void par_ranges(size_t n, size_t parts, F f) {
    size_t per = (n + parts - 1) / parts;
    if (per == 0) per = 1;
    std::vector<std::thread> th;
    for (size_t s = 0; s < n; s += per) {
        size_t e = s + per < n ? s + per : n;
        th.emplace_back([=] { f(s, e); });
    }
    for (auto& t : th) t.join();
}

inline Shape broadcast_shape(const Shape& a, const Shape& b) {
    if (a.size() != b.size()) fail("broadcast: rank mismatch");
    Shape o(a.size());
    for (size_t i = 0; i < a.size(); i++) {
        if (a[i] == b[i]) o[i] = a[i];
        else if (a[i] == 1) o[i] = b[i];
        else if (b[i] == 1) o[i] = a[i];
        else fail("broadcast: incompatible shapes");
    }
    return o;
}

inline std::vector<size_t> broadcast_strides(const Shape& sh, const Shape& out) {
    std::vector<size_t> st(out.size(), 0);
    size_t acc = 1;
    for (size_t i = out.size(); i-- > 0;) {
        st[i] = sh[i] == 1 ? 0 : acc;
        acc *= sh[i];
    }
    return st;
}

// Row-major walk of `out`, calling f(offset_a, offset_b).
template <class F>
inline void for_each_offset2(const Shape& out, const std::vector<size_t>& sa, const std::vector<size_t>& sb, F f) {
    size_t rank = out.size();
    size_t n = numel(out);
    if (n == 0) return;
    if (rank == 0) { f(0, 0); return; }
    std::vector<size_t> idx(rank, 0);
    size_t last = out[rank - 1];
    size_t ba = 0, bb = 0;
    for (;;) {
        for (size_t j = 0; j < last; j++) f(ba + j * sa[rank - 1], bb + j * sb[rank - 1]);
        size_t d = rank - 1;
        for (;;) {
            if (d == 0) return;
            d--;
            idx[d]++;
            ba += sa[d];
            bb += sb[d];
            if (idx[d] < out[d]) break;
            ba -= sa[d] * idx[d];
            bb -= sb[d] * idx[d];
            idx[d] = 0;
        }
    }
}

struct Bool {
    std::shared_ptr<std::vector<uint8_t>> v;
    Shape sh;
    Bool() {}
    Bool(std::vector<uint8_t> d, Shape s) : v(std::make_shared<std::vector<uint8_t>>(std::move(d))), sh(std::move(s)) {}
    Bool bool_not() const {
        std::vector<uint8_t> o(v->size());
        for (size_t i = 0; i < o.size(); i++) o[i] = !(*v)[i];
        return Bool(std::move(o), sh);
    }
};

struct Int {
    std::vector<int64_t> v;
    Shape sh;
};

template <class T>
struct Engine {
    struct Tensor;
    typedef std::function<std::vector<std::optional<Tensor>>(const Tensor&, const std::vector<bool>&)> BackwardFn;

    struct Node {
        uint64_t id;
        size_t order;
        std::vector<std::shared_ptr<Node>> inputs;  // null where an input is not tracked
        BackwardFn backward;                        // empty for a leaf
        bool leaf;
    };

    static uint64_t next_id() {
        static uint64_t n = 0;
        return n++;
    }

    struct Tensor {
        std::shared_ptr<const std::vector<T>> st;
        Shape sh;
        size_t order = 0;
        std::shared_ptr<Node> node;

        Tensor() {}
        Tensor(std::vector<T> d, Shape s) : st(std::make_shared<const std::vector<T>>(std::move(d))), sh(std::move(s)) {
            if (st->size() != numel(sh)) fail("tensor: data does not match shape");
        }
        static Tensor from_f64s(const double* p, Shape s) {
            size_t n = numel(s);
            std::vector<T> d(n);
            for (size_t i = 0; i < n; i++) d[i] = (T)p[i];
            return Tensor(std::move(d), std::move(s));
        }
        static Tensor full(Shape s, double x) { return Tensor(std::vector<T>(numel(s), (T)x), s); }

        const std::vector<T>& v() const { return *st; }
        size_t n() const { return st->size(); }
        size_t rank() const { return sh.size(); }

        Tensor untracked() const {
            Tensor t;
            t.st = st;
            t.sh = sh;
            return t;
        }
        Tensor detach() const { return untracked(); }
        Tensor require_grad() const {
            Tensor t = untracked();
            t.node = std::make_shared<Node>(Node{next_id(), 0, {}, BackwardFn(), true});
            return t;
        }
    };

    // ------------------------------------------------------------------ backend kernels

    template <class F>
    static std::vector<T> be_map(const std::vector<T>& x, F f) {
        std::vector<T> o(x.size());
        const Config& c = config();
        if (c.mode == CpuMode::Fast && x.size() >= FAST_MIN_MAP && c.threads > 1) {
            par_ranges(x.size(), (size_t)c.threads, [&](size_t s, size_t e) { for (size_t i = s; i < e; i++) o[i] = f(x[i]); });
        } else {
            for (size_t i = 0; i < x.size(); i++) o[i] = f(x[i]);
        }
        return o;
    }

    template <class F>
    static std::pair<std::vector<T>, Shape> be_zip(const std::vector<T>& a, const Shape& ash, const std::vector<T>& b, const Shape& bsh, F f) {
        if (ash == bsh) {
            std::vector<T> o(a.size());
            const Config& c = config();
            if (c.mode == CpuMode::Fast && a.size() >= FAST_MIN_ZIP && c.threads > 1) {
                par_ranges(a.size(), (size_t)c.threads, [&](size_t s, size_t e) { for (size_t i = s; i < e; i++) o[i] = f(a[i], b[i]); });
            } else {
                for (size_t i = 0; i < a.size(); i++) o[i] = f(a[i], b[i]);
            }
            return {std::move(o), ash};
        }
        // The broadcast path is single-threaded on both backends (src/tensor/backend.rs:158).
        Shape out = broadcast_shape(ash, bsh);
        auto sa = broadcast_strides(ash, out), sb = broadcast_strides(bsh, out);
        std::vector<T> o;
        o.reserve(numel(out));
        for_each_offset2(out, sa, sb, [&](size_t oa, size_t ob) { o.push_back(f(a[oa], b[ob])); });
        return {std::move(o), out};
    }

    static T unrolled_sum(const T* xs, size_t len) {
        T acc = 0;
        T p0 = 0, p1 = 0, p2 = 0, p3 = 0, p4 = 0, p5 = 0, p6 = 0, p7 = 0;
        while (len >= 8) {
            p0 = p0 + xs[0];
            p1 = p1 + xs[1];
            p2 = p2 + xs[2];
            p3 = p3 + xs[3];
            p4 = p4 + xs[4];
            p5 = p5 + xs[5];
            p6 = p6 + xs[6];
            p7 = p7 + xs[7];
            xs += 8;
            len -= 8;
        }
        acc = acc + (p0 + p4);
        acc = acc + (p1 + p5);
        acc = acc + (p2 + p6);
        acc = acc + (p3 + p7);
        for (size_t i = 0; i < len && i < 7; i++) acc = acc + xs[i];
        return acc;
    }

    static T simd_sum(const T* xs, size_t len) {
        T acc[16];
        for (int i = 0; i < 16; i++) acc[i] = 0;
        size_t full = len / 16 * 16;
        for (size_t c = 0; c < full; c += 16)
            for (int i = 0; i < 16; i++) acc[i] = acc[i] + xs[c + i];
        T total = 0;
        for (int i = 0; i < 16; i++) total = total + acc[i];
        for (size_t i = full; i < len; i++) total = total + xs[i];
        return total;
    }

    static std::pair<std::vector<T>, Shape> ref_sum_dim(const T* x, const Shape& sh, size_t dim) {
        Shape out_sh = sh;
        out_sh[dim] = 1;
        size_t n = sh[dim], outer = 1, inner = 1;
        for (size_t i = 0; i < dim; i++) outer *= sh[i];
        for (size_t i = dim + 1; i < sh.size(); i++) inner *= sh[i];
        if (dim + 1 == sh.size()) {
            std::vector<T> v(outer);
            for (size_t o = 0; o < outer; o++) v[o] = unrolled_sum(x + o * n, n);
            return {std::move(v), out_sh};
        }
        std::vector<T> v(outer * inner, (T)0);
        for (size_t o = 0; o < outer; o++)
            for (size_t k = 0; k < n; k++) {
                const T* row = x + (o * n + k) * inner;
                T* acc = v.data() + o * inner;
                for (size_t i = 0; i < inner; i++) acc[i] = acc[i] + row[i];
            }
        return {std::move(v), out_sh};
    }

    static std::pair<std::vector<T>, Shape> be_sum_dim(const std::vector<T>& x, const Shape& sh, size_t dim) {
        const Config& c = config();
        if (!(c.mode == CpuMode::Fast && x.size() >= FAST_MIN_SUM && c.threads > 1)) return ref_sum_dim(x.data(), sh, dim);
        Shape out_sh = sh;
        out_sh[dim] = 1;
        size_t n = sh[dim];
        size_t parts = (size_t)c.threads;
        if (dim + 1 == sh.size() && n > 0) {
            size_t lanes = x.size() / n;
            std::vector<T> v(lanes, (T)0);
            par_ranges(lanes, parts, [&](size_t s, size_t e) { for (size_t l = s; l < e; l++) v[l] = simd_sum(x.data() + l * n, n); });
            return {std::move(v), out_sh};
        }
        size_t outer = 1, inner = 1;
        for (size_t i = 0; i < dim; i++) outer *= sh[i];
        for (size_t i = dim + 1; i < sh.size(); i++) inner *= sh[i];
        std::vector<T> v(outer * inner, (T)0);
        par_ranges(outer, parts, [&](size_t s, size_t e) {
            auto part = ref_sum_dim(x.data() + s * n * inner, Shape{e - s, n, inner}, 1);
            for (size_t i = 0; i < part.first.size(); i++) v[s * inner + i] = part.first[i];
        });
        return {std::move(v), out_sh};
    }

    static T be_sum_all(const std::vector<T>& x) {
        const Config& c = config();
        if (c.mode == CpuMode::Fast && x.size() >= FAST_MIN_SUM) return simd_sum(x.data(), x.size());
        return unrolled_sum(x.data(), x.size());
    }

    static std::pair<std::vector<int64_t>, Shape> argmax_dim(const std::vector<T>& x, const Shape& sh, size_t dim) {
        Shape out_sh = sh;
        out_sh[dim] = 1;
        size_t n = sh[dim], outer = 1, inner = 1;
        for (size_t i = 0; i < dim; i++) outer *= sh[i];
        for (size_t i = dim + 1; i < sh.size(); i++) inner *= sh[i];
        std::vector<int64_t> v;
        v.reserve(outer * inner);
        for (size_t o = 0; o < outer; o++)
            for (size_t i = 0; i < inner; i++) {
                auto at = [&](size_t k) { return x[(o * n + k) * inner + i]; };
                T best = at(0);
                size_t idx = 0;
                for (size_t k = 0; k < n; k++) {
                    T e = at(k);
                    if (best != best) break;
                    if (e != e || e > best) {
                        best = e;
                        idx = k;
                    }
                }
                v.push_back((int64_t)idx);
            }
        return {std::move(v), out_sh};
    }

    static std::vector<T> k_gather(const std::vector<T>& x, const Shape& sh, size_t dim, const std::vector<int64_t>& idx, const Shape& ish) {
        size_t n = sh[dim], m = ish[dim], outer = 1, inner = 1;
        for (size_t i = 0; i < dim; i++) outer *= ish[i];
        for (size_t i = dim + 1; i < ish.size(); i++) inner *= ish[i];
        std::vector<T> v;
        v.reserve(idx.size());
        for (size_t o = 0; o < outer; o++)
            for (size_t k = 0; k < m; k++)
                for (size_t i = 0; i < inner; i++) {
                    int64_t j = idx[(o * m + k) * inner + i];
                    if (j < 0 || (size_t)j >= n) fail("gather index out of range");
                    v.push_back(x[(o * n + (size_t)j) * inner + i]);
                }
        return v;
    }

    static std::vector<T> scatter_add_zeros(const Shape& sh, size_t dim, const std::vector<int64_t>& idx, const Shape& ish, const std::vector<T>& vals) {
        size_t n = sh[dim], m = ish[dim], outer = 1, inner = 1;
        for (size_t i = 0; i < dim; i++) outer *= ish[i];
        for (size_t i = dim + 1; i < ish.size(); i++) inner *= ish[i];
        std::vector<T> out(numel(sh), (T)0);
        for (size_t o = 0; o < outer; o++)
            for (size_t k = 0; k < m; k++)
                for (size_t i = 0; i < inner; i++) {
                    size_t p = (o * m + k) * inner + i;
                    size_t j = (size_t)idx[p];
                    T& t = out[(o * n + j) * inner + i];
                    t = t + vals[p];
                }
        return out;
    }

    // ------------------------------------------------------------------ tape

    static Tensor record(std::vector<T> data, Shape shape, std::initializer_list<const Tensor*> inputs, std::function<BackwardFn(const Tensor&)> backward) {
        Tensor out(std::move(data), std::move(shape));
        return attach(out, inputs, backward);
    }

    static Tensor attach(Tensor out, std::initializer_list<const Tensor*> inputs, std::function<BackwardFn(const Tensor&)> backward) {
        size_t order = 0;
        bool tracked = false;
        for (const Tensor* t : inputs) {
            if (t->order > order) order = t->order;
            if (t->node) tracked = true;
        }
        order += 1;
        out.order = order;
        out.node = nullptr;
        if (tracked) {
            Tensor saved = out.untracked();
            auto n = std::make_shared<Node>();
            n->id = next_id();
            n->order = order;
            for (const Tensor* t : inputs) n->inputs.push_back(t->node);
            n->backward = backward(saved);
            n->leaf = false;
            out.node = n;
        }
        return out;
    }

    typedef std::vector<std::optional<Tensor>> Grads;

    static Tensor unbroadcast(Tensor g, const Shape& shape) {
        Shape gs = g.sh;
        for (size_t i = 0; i < gs.size(); i++)
            if (gs[i] != shape[i]) {
                if (shape[i] != 1) fail("invalid broadcast in backward");
                g = sum_dim(g, i);
            }
        return g;
    }

    // ------------------------------------------------------------------ ops

    static Tensor add_raw(const Tensor& a, const Tensor& b) {
        auto r = be_zip(a.v(), a.sh, b.v(), b.sh, [](T x, T y) { return x + y; });
        return Tensor(std::move(r.first), r.second);
    }

    static Tensor add(const Tensor& a, const Tensor& b) {
        auto r = be_zip(a.v(), a.sh, b.v(), b.sh, [](T x, T y) { return x + y; });
        Shape ls = a.sh, rs = b.sh;
        return record(std::move(r.first), r.second, {&a, &b}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>& n) {
                Grads o(2);
                if (n[0]) o[0] = unbroadcast(g, ls);
                if (n[1]) o[1] = unbroadcast(g, rs);
                return o;
            };
        });
    }

    static Tensor sub(const Tensor& a, const Tensor& b) {
        auto r = be_zip(a.v(), a.sh, b.v(), b.sh, [](T x, T y) { return x - y; });
        Shape ls = a.sh, rs = b.sh;
        return record(std::move(r.first), r.second, {&a, &b}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>& n) {
                Grads o(2);
                if (n[0]) o[0] = unbroadcast(g, ls);
                if (n[1]) o[1] = unbroadcast(neg(g), rs);
                return o;
            };
        });
    }

    static Tensor mul(const Tensor& a, const Tensor& b) {
        auto r = be_zip(a.v(), a.sh, b.v(), b.sh, [](T x, T y) { return x * y; });
        Shape ls = a.sh, rs = b.sh;
        Tensor l = a.untracked(), rr = b.untracked();
        return record(std::move(r.first), r.second, {&a, &b}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>& n) {
                Grads o(2);
                if (n[0]) o[0] = unbroadcast(mul(g, rr), ls);
                if (n[1]) o[1] = unbroadcast(mul(g, l), rs);
                return o;
            };
        });
    }

    static Tensor div(const Tensor& a, const Tensor& b) {
        auto r = be_zip(a.v(), a.sh, b.v(), b.sh, [](T x, T y) { return x / y; });
        Shape ls = a.sh, rs = b.sh;
        Tensor l = a.untracked(), rr = b.untracked();
        return record(std::move(r.first), r.second, {&a, &b}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>& n) {
                Grads o(2);
                if (n[0]) o[0] = unbroadcast(div(g, rr), ls);
                if (n[1]) o[1] = unbroadcast(mul(neg(g), div(div(l, rr), rr)), rs);
                return o;
            };
        });
    }

    static Tensor add_scalar(const Tensor& a, double s64) {
        T s = (T)s64;
        return record(be_map(a.v(), [s](T x) { return x + s; }), a.sh, {&a}, [](const Tensor&) {
            return [](const Tensor& g, const std::vector<bool>&) { return Grads{g}; };
        });
    }
    static Tensor sub_scalar(const Tensor& a, double s64) {
        T s = (T)s64;
        return record(be_map(a.v(), [s](T x) { return x - s; }), a.sh, {&a}, [](const Tensor&) {
            return [](const Tensor& g, const std::vector<bool>&) { return Grads{g}; };
        });
    }
    static Tensor mul_scalar(const Tensor& a, double s64) {
        T s = (T)s64;
        return record(be_map(a.v(), [s](T x) { return x * s; }), a.sh, {&a}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>&) { return Grads{mul_scalar(g, s64)}; };
        });
    }
    static Tensor div_scalar(const Tensor& a, double s64) {
        T s = (T)s64;
        return record(be_map(a.v(), [s](T x) { return x / s; }), a.sh, {&a}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>&) { return Grads{div_scalar(g, s64)}; };
        });
    }
    static Tensor neg(const Tensor& a) {
        return record(be_map(a.v(), [](T x) { return -x; }), a.sh, {&a}, [](const Tensor&) {
            return [](const Tensor& g, const std::vector<bool>&) { return Grads{neg(g)}; };
        });
    }
    static Tensor exp(const Tensor& a) {
        return record(be_map(a.v(), [](T x) { return (T)std::exp(x); }), a.sh, {&a}, [](const Tensor& y) {
            return [y](const Tensor& g, const std::vector<bool>&) { return Grads{mul(g, y)}; };
        });
    }
    static Tensor log(const Tensor& a) {
        Tensor x = a.untracked();
        return record(be_map(a.v(), [](T x) { return (T)std::log(x); }), a.sh, {&a}, [x](const Tensor&) {
            return [x](const Tensor& g, const std::vector<bool>&) { return Grads{div(g, x)}; };
        });
    }
    static Tensor sign(const Tensor& a) {
        return record(be_map(a.v(), [](T x) { return x == (T)0 ? (T)0 : (std::signbit(x) ? (T)-1 : (T)1); }), a.sh, {&a}, [](const Tensor&) {
            return [](const Tensor& g, const std::vector<bool>&) { return Grads{Tensor::full(g.sh, 0.0)}; };
        });
    }
    static Tensor abs(const Tensor& a) {
        Tensor x = a.untracked();
        return record(be_map(a.v(), [](T x) { return (T)std::fabs(x); }), a.sh, {&a}, [x](const Tensor&) {
            return [x](const Tensor& g, const std::vector<bool>&) { return Grads{mul(g, sign(x))}; };
        });
    }

    // comparisons against a scalar (untracked); the scalar is converted to the tensor's dtype
    template <class F>
    static Bool cmp(const Tensor& a, double s64, F f) {
        T s = (T)s64;
        std::vector<uint8_t> o(a.n());
        for (size_t i = 0; i < o.size(); i++) o[i] = f(a.v()[i], s) ? 1 : 0;
        return Bool(std::move(o), a.sh);
    }
    static Bool greater_elem(const Tensor& a, double s) { return cmp(a, s, [](T x, T y) { return x > y; }); }
    static Bool lower_elem(const Tensor& a, double s) { return cmp(a, s, [](T x, T y) { return x < y; }); }
    static Bool equal_elem(const Tensor& a, double s) { return cmp(a, s, [](T x, T y) { return x == y; }); }

    static Tensor float_of(const Bool& b) {
        std::vector<T> o(b.v->size());
        for (size_t i = 0; i < o.size(); i++) o[i] = (*b.v)[i] ? (T)1 : (T)0;
        return Tensor(std::move(o), b.sh);
    }

    static std::vector<uint8_t> broadcast_bool(const Bool& m, const Shape& out) {
        if (m.sh == out) return *m.v;
        if (m.sh.size() != out.size()) fail("mask_fill: mask rank");
        auto st = broadcast_strides(m.sh, out);
        std::vector<uint8_t> o;
        o.reserve(numel(out));
        for_each_offset2(out, st, st, [&](size_t a, size_t) { o.push_back((*m.v)[a]); });
        return o;
    }

    static Tensor mask_fill(const Tensor& a, const Bool& mask, double value64) {
        T value = (T)value64;
        std::vector<uint8_t> m = broadcast_bool(mask, a.sh);
        std::vector<T> o(a.n());
        for (size_t i = 0; i < o.size(); i++) o[i] = m[i] ? value : a.v()[i];
        Bool full(std::move(m), a.sh);
        return record(std::move(o), a.sh, {&a}, [full](const Tensor&) {
            return [full](const Tensor& g, const std::vector<bool>&) { return Grads{mask_fill(g, full, 0.0)}; };
        });
    }

    static Tensor clamp_min(const Tensor& a, double mn) { return mask_fill(a, lower_elem(a, mn), mn); }
    static Tensor clamp_max(const Tensor& a, double mx) { return mask_fill(a, greater_elem(a, mx), mx); }
    static Tensor clamp(const Tensor& a, double mn, double mx) { return clamp_min(clamp_max(a, mx), mn); }

    static Tensor sum(const Tensor& a) {
        Shape shape = a.sh;
        return record(std::vector<T>{be_sum_all(a.v())}, Shape{1}, {&a}, [shape](const Tensor&) {
            return [shape](const Tensor& g, const std::vector<bool>&) {
                Tensor val = Tensor::full(shape, 1.0);
                Tensor gr = reshape(g, Shape(shape.size(), 1));
                return Grads{mul(val, gr)};
            };
        });
    }

    static Tensor sum_dim(const Tensor& a, size_t dim) {
        if (dim >= a.sh.size()) fail("sum_dim: dim out of range");
        auto r = be_sum_dim(a.v(), a.sh, dim);
        Shape shape = a.sh;
        return record(std::move(r.first), r.second, {&a}, [shape, dim](const Tensor&) {
            return [shape, dim](const Tensor& g, const std::vector<bool>&) {
                Tensor ones = Tensor::full(shape, 1.0);
                Tensor gs = sum_dim(g, dim);
                return Grads{mul(ones, gs)};
            };
        });
    }

    // src/tensor/float.rs:683-706: the lane sum divided by the lane's length; backward
    // ones · g.sum_dim(dim) / n.
    static Tensor mean_dim(const Tensor& a, size_t dim) {
        if (dim >= a.sh.size()) fail("mean_dim: dim out of range");
        auto r = be_sum_dim(a.v(), a.sh, dim);
        const T n = (T)a.sh[dim];
        for (T& x : r.first) x = x / n;
        Shape shape = a.sh;
        return record(std::move(r.first), r.second, {&a}, [shape, dim](const Tensor&) {
            return [shape, dim](const Tensor& g, const std::vector<bool>&) {
                Tensor ones = Tensor::full(shape, 1.0);
                Tensor gs = sum_dim(g, dim);
                return Grads{div_scalar(mul(ones, gs), (double)shape[dim])};
            };
        });
    }

    // IntTensor::one_hot_float (src/tensor/int.rs:214-222): an untracked 0/1 tensor with one more axis.
    static Tensor one_hot(const Int& idx, size_t n) {
        std::vector<T> d(idx.v.size() * n, (T)0);
        for (size_t i = 0; i < idx.v.size(); i++) {
            if (idx.v[i] < 0 || (size_t)idx.v[i] >= n) fail("one_hot: index outside 0..n");
            d[i * n + (size_t)idx.v[i]] = (T)1;
        }
        Shape sh = idx.sh;
        sh.push_back(n);
        return Tensor(std::move(d), sh);
    }

    static Tensor max_dim(const Tensor& a, size_t dim) {
        auto am = argmax_dim(a.v(), a.sh, dim);
        std::vector<T> vals = k_gather(a.v(), a.sh, dim, am.first, am.second);
        Shape shape = a.sh, ish = am.second;
        std::vector<int64_t> idx = am.first;
        return record(std::move(vals), ish, {&a}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>&) { return Grads{Tensor(scatter_add_zeros(shape, dim, idx, ish, g.v()), shape)}; };
        });
    }

    static Int argmax(const Tensor& a, size_t dim) {
        auto am = argmax_dim(a.v(), a.sh, dim);
        return Int{am.first, am.second};
    }

    static Tensor gather(const Tensor& a, size_t dim, const Int& indices) {
        std::vector<T> vals = k_gather(a.v(), a.sh, dim, indices.v, indices.sh);
        Shape shape = a.sh;
        Int ind = indices;
        return record(std::move(vals), indices.sh, {&a}, [=](const Tensor&) {
            return [=](const Tensor& g, const std::vector<bool>&) { return Grads{Tensor(scatter_add_zeros(shape, dim, ind.v, ind.sh, g.v()), shape)}; };
        });
    }

    // A view in the reference (record_view): same storage, new shape, order + 1.
    static Tensor reshape(const Tensor& a, Shape shape) {
        if (numel(shape) != a.n()) fail("reshape: element count");
        Tensor out;
        out.st = a.st;
        out.sh = shape;
        out.order = a.order + 1;
        if (a.node) {
            Shape original = a.sh;
            auto n = std::make_shared<Node>();
            n->id = next_id();
            n->order = out.order;
            n->inputs.push_back(a.node);
            n->backward = [original](const Tensor& g, const std::vector<bool>&) { return Grads{reshape(g, original)}; };
            n->leaf = false;
            out.node = n;
        }
        return out;
    }

    // expand (src/tensor/float.rs:816-841): a broadcast view; here the values are materialised.
    static Tensor expand(const Tensor& a, Shape out_sh) {
        size_t ni = a.sh.size(), no = out_sh.size();
        Shape aligned(no, 1);
        for (size_t i = 0; i < ni; i++) aligned[no - ni + i] = a.sh[i];
        auto st = broadcast_strides(aligned, out_sh);
        std::vector<T> o;
        o.reserve(numel(out_sh));
        for_each_offset2(out_sh, st, st, [&](size_t x, size_t) { o.push_back(a.v()[x]); });
        Tensor out(std::move(o), out_sh);
        out.order = a.order + 1;
        if (a.node) {
            Shape shape_in = a.sh;
            auto n = std::make_shared<Node>();
            n->id = next_id();
            n->order = out.order;
            n->inputs.push_back(a.node);
            n->backward = [=](const Tensor& g0, const std::vector<bool>&) {
                Tensor g = g0;
                Shape gs = g.sh;
                for (size_t i = 0; i < no; i++)
                    if (aligned[i] == 1 && gs[i] != 1) g = sum_dim(g, i);
                return Grads{reshape(g, shape_in)};
            };
            n->leaf = false;
            out.node = n;
        }
        return out;
    }

    // log_softmax (src/tensor/activation.rs:30-42)
    static Tensor log_softmax(const Tensor& x, size_t dim) {
        Tensor xu = x.untracked();
        Tensor mx = max_dim(xu, dim);
        Tensor shifted = sub(xu, mx);
        Tensor lse = log(sum_dim(exp(shifted), dim));
        Tensor y = sub(shifted, lse);
        return attach(y.untracked(), {&x}, [dim](const Tensor& ys) {
            return [ys, dim](const Tensor& g, const std::vector<bool>&) {
                Tensor s = sum_dim(g, dim);
                return Grads{sub(g, mul(exp(ys), s))};
            };
        });
    }

    // softmax (src/tensor/activation.rs:15-26): exp(x − max) / Σ exp(x − max); backward
    // y · (g − Σ g·y) from the saved output
    static Tensor softmax(const Tensor& x, size_t dim) {
        Tensor xu = x.untracked();
        Tensor mx = max_dim(xu, dim);
        Tensor e = exp(sub(xu, mx));
        Tensor y = div(e, sum_dim(e, dim));
        return attach(y.untracked(), {&x}, [dim](const Tensor& ys) {
            return [ys, dim](const Tensor& g, const std::vector<bool>&) {
                Tensor s = sum_dim(mul(g, ys), dim);
                return Grads{mul(ys, sub(g, s))};
            };
        });
    }

    // logsumexp (src/tensor/activation.rs:71-77): m + log Σ exp(x − m) with the shift 0 where the
    // lane's maximum is ±inf; backward g · exp(x − out)
    static Tensor logsumexp(const Tensor& x, size_t dim) {
        Tensor xu = x.untracked();
        Tensor m = max_dim(xu, dim);
        m = mask_fill(m, equal_elem(abs(m), INFINITY), 0.0).untracked();
        Tensor out = add(log(sum_dim(exp(sub(xu, m)), dim)), m);
        return attach(out.untracked(), {&x}, [xu](const Tensor& ys) {
            return [ys, xu](const Tensor& g, const std::vector<bool>&) { return Grads{mul(g, exp(sub(xu, ys)))}; };
        });
    }

    // ------------------------------------------------------------------ backward

    struct Gradients {
        std::unordered_map<uint64_t, Tensor> map;
        const Tensor* get(const Tensor& t) const {
            if (!t.node) return nullptr;
            auto it = map.find(t.node->id);
            return it == map.end() ? nullptr : &it->second;
        }
    };

    static Gradients backward(const Tensor& root) {
        if (!root.node) fail("backward: the root is not tracked");
        if (root.n() != 1) fail("backward: the root must have one element");
        std::shared_ptr<Node> root_node = root.node;
        std::unordered_map<uint64_t, std::shared_ptr<Node>> steps;
        {
            std::vector<std::shared_ptr<Node>> stack{root_node};
            while (!stack.empty()) {
                auto n = stack.back();
                stack.pop_back();
                if (steps.count(n->id)) continue;
                for (auto& p : n->inputs)
                    if (p) stack.push_back(p);
                steps[n->id] = n;
            }
        }
        std::vector<std::vector<std::shared_ptr<Node>>> tape(root_node->order + 1);
        std::unordered_set<uint64_t> visited;
        visited.insert(root_node->id);
        std::vector<uint64_t> parents;
        for (auto& p : root_node->inputs)
            if (p) parents.push_back(p->id);
        steps.erase(root_node->id);
        tape[root_node->order].push_back(root_node);
        while (!parents.empty()) {
            uint64_t id = parents.back();
            parents.pop_back();
            auto it = steps.find(id);
            if (it == steps.end()) continue;
            auto step = it->second;
            steps.erase(it);
            if (visited.count(step->id)) continue;
            visited.insert(step->id);
            for (auto& p : step->inputs)
                if (p && !visited.count(p->id)) parents.push_back(p->id);
            if (step->order < tape.size()) tape[step->order].push_back(step);
        }
        Gradients out;
        auto& grads = out.map;
        grads[root_node->id] = Tensor::full(root.sh, 1.0);
        for (size_t lvl = tape.size(); lvl-- > 0;) {
            for (auto& node : tape[lvl]) {
                if (node->leaf) continue;
                auto git = grads.find(node->id);
                if (git == grads.end()) fail("a node's gradient is recorded before its step runs");
                Tensor grad = git->second;
                grads.erase(git);
                std::vector<bool> needs;
                for (auto& i : node->inputs) needs.push_back((bool)i);
                Grads outs = node->backward(grad, needs);
                for (size_t k = 0; k < node->inputs.size(); k++) {
                    auto& input = node->inputs[k];
                    if (!input) continue;
                    if (!outs[k]) fail("a tracked input receives a gradient");
                    Tensor g = *outs[k];
                    auto old = grads.find(input->id);
                    if (old != grads.end()) {
                        g = add_raw(g, old->second);
                        grads.erase(old);
                    }
                    grads[input->id] = g.untracked();
                }
            }
        }
        return out;
    }
};

}  // namespace orc
