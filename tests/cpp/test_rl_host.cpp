// GPU tests of the C++ host mirror of `nn::rl` (noetic_tensor_b200/host/noetic_rl.hpp), written
// the way the reference's own tests are (src/nn/tests/rl.rs): every function against an f64
// restatement on the host, hand-computed reductions, the masking edges, the gradients against
// closed forms. Run by tests/test_gpu_host_cpp.py; exits non-zero on the first failed check.
#include <algorithm>
#include <cstdio>
#include <limits>
#include <random>

#include "../../noetic_tensor_b200/host/noetic_loss.hpp"

using namespace noetic;
namespace rl = noetic::nn::rl;
using rl::TokenReduction;

static int g_checks = 0;
#define CHECK(cond, ...)                                                \
    do {                                                                \
        g_checks++;                                                     \
        if (!(cond)) {                                                  \
            std::printf("FAILED %s:%d: %s\n  ", __FILE__, __LINE__, #cond); \
            std::printf(__VA_ARGS__);                                   \
            std::printf("\n");                                          \
            std::exit(1);                                               \
        }                                                               \
    } while (0)

static void close_all(const std::vector<float>& got, const std::vector<double>& want, double tol, const char* what) {
    CHECK(got.size() == want.size(), "%s: %zu values, expected %zu", what, got.size(), want.size());
    for (size_t i = 0; i < got.size(); i++) {
        double e = std::fabs((double)got[i] - want[i]) / (1.0 + std::fabs(want[i]));
        if ((double)got[i] == want[i]) e = 0.0;
        CHECK(e <= tol, "%s[%zu]: got %.9g, want %.9g (error %.3e > %.1e)", what, i, (double)got[i], want[i], e, tol);
    }
}

template <class F>
static bool throws(F f, const char* needle) {
    try {
        f();
    } catch (const std::exception& e) {
        return std::string(e.what()).find(needle) != std::string::npos;
    }
    return false;
}

// ---- f64 host restatement ----------------------------------------------------------------------
struct Case {
    size_t S = 2, B = 3, T = 4, V = 37;
    std::vector<float> logits;  // values exactly representable in the storage dtype
    std::vector<int64_t> tokens;
    std::vector<float> mask;
    size_t n() const { return S * B * T; }
    Shape sh() const { return Shape{S, B, T}; }
    Shape lsh() const { return Shape{S, B, T, V}; }
};
static float through_bf16(float x) {
    uint32_t b = (uint32_t)bf16_from_f32(x) << 16;
    float y;
    std::memcpy(&y, &b, 4);
    return y;
}
static Case make_case(unsigned seed, double lo, double hi, bool bf16, size_t V = 37) {
    Case c;
    c.V = V;
    std::mt19937_64 g(seed);
    std::uniform_real_distribution<double> u(lo, hi), u01(0.0, 1.0);
    c.logits.resize(c.n() * V);
    for (float& x : c.logits) {
        x = (float)u(g);
        if (bf16) x = through_bf16(x);
    }
    for (size_t i = 0; i < c.n(); i++) c.tokens.push_back((int64_t)(g() % V));
    for (size_t i = 0; i < c.n(); i++) c.mask.push_back(u01(g) < 0.7 ? 1.f : 0.f);
    c.mask[0] = 1.f;
    for (size_t t = 0; t < c.T; t++) c.mask[c.T + t] = 0.f;  // a sequence with no scored position
    return c;
}
// log-softmax of one row at temperature tau with an optional allow mask
static std::vector<double> log_softmax_row(const float* z, size_t V, double tau = 1.0, const uint8_t* allow = nullptr) {
    std::vector<double> y(V);
    double m = -INFINITY;
    for (size_t v = 0; v < V; v++) {
        y[v] = (allow && !allow[v]) ? -INFINITY : (double)(float)((float)z[v] / (float)tau);
        m = std::max(m, y[v]);
    }
    double s = 0.0;
    for (size_t v = 0; v < V; v++) s += std::exp(y[v] - m);
    for (size_t v = 0; v < V; v++) y[v] = y[v] - m - std::log(s);
    return y;
}
static std::vector<double> reduce_host(const std::vector<double>& per, const std::vector<float>& mask, size_t S, size_t B, size_t T, TokenReduction r) {
    std::vector<double> out;
    if (r == TokenReduction::None) return per;
    for (size_t s = 0; s < S; s++) {
        double sum = 0, cnt = 0, seqsum = 0, seqs = 0;
        for (size_t b = 0; b < B; b++) {
            double bs = 0, bc = 0;
            for (size_t t = 0; t < T; t++) {
                size_t i = (s * B + b) * T + t;
                bs += per[i];
                bc += mask.empty() ? 1.0 : mask[i];
            }
            sum += bs;
            cnt += bc;
            double ps = bs / std::max(bc, 1.0);
            if (r == TokenReduction::PerSequence) out.push_back(ps);
            seqsum += ps;
            seqs += bc > 0 ? 1.0 : 0.0;
        }
        if (r == TokenReduction::Sum) out.push_back(sum);
        if (r == TokenReduction::TokenMean) out.push_back(sum / std::max(cnt, 1.0));
        if (r == TokenReduction::SequenceMean) out.push_back(seqsum / std::max(seqs, 1.0));
    }
    return out;
}
static const TokenReduction kReductions[] = {TokenReduction::None, TokenReduction::Sum, TokenReduction::TokenMean, TokenReduction::PerSequence, TokenReduction::SequenceMean};

static Device dev = Device::Cuda(0);

// ---- token_log_probs (src/nn/tests/rl.rs:100-156) ----------------------------------------------
static void test_token_log_probs() {
    for (int bf = 0; bf < 2; bf++) {
        Case c = make_case(800 + bf, -6.0, 6.0, bf);
        Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, bf ? DType::BF16 : DType::F32).require_grad();
        IntTensor tok = IntTensor::from_data(c.tokens, c.sh());
        Tensor lp = rl::token_log_probs(z, tok);
        CHECK(lp.shape() == c.sh(), "shape");
        std::vector<double> want, gwant(c.n() * c.V);
        for (size_t i = 0; i < c.n(); i++) {
            auto y = log_softmax_row(&c.logits[i * c.V], c.V);
            want.push_back(y[c.tokens[i]]);
            for (size_t v = 0; v < c.V; v++) gwant[i * c.V + v] = ((int64_t)v == c.tokens[i] ? 1.0 : 0.0) - std::exp(y[v]);
        }
        close_all(lp.to_vec(), want, 1e-6, "token_log_probs");
        Gradients g = backward(lp);
        const Tensor* d = g.grad(z);
        CHECK(d != nullptr && d->shape() == c.lsh(), "gradient of the logits");
        close_all(d->to_vec(), gwant, 1e-6, "d token_log_probs");
    }
    // large and excluded logits: no overflow, −∞ log-prob of an excluded token, zero gradient there
    {
        std::vector<float> l = {1e4f, -1e4f, 0.f, 1e3f, -1e4f, -1e4f, 1e4f, 1e4f};
        Tensor z = Tensor::from_f32(l, Shape{1, 1, 2, 4}, dev).require_grad();
        Tensor lp = rl::token_log_probs(z, IntTensor::from_data({0, 2}, Shape{1, 1, 2}));
        auto v = lp.to_vec();
        CHECK(std::fabs(v[0]) < 1e-6 && std::fabs(v[1] - std::log(0.5)) < 1e-6, "%g %g", v[0], v[1]);
        close_all(backward(lp).grad(z)->to_vec(), {0, 0, 0, 0, 0, 0, 0.5, -0.5}, 1e-6, "d large logits");
        std::vector<float> row = {1.f, -INFINITY, 0.f, 2.f, 1.f, -INFINITY, 0.f, 2.f};
        Tensor z2 = Tensor::from_f32(row, Shape{1, 1, 2, 4}, dev).require_grad();
        Tensor lp2 = rl::token_log_probs(z2, IntTensor::from_data({1, 3}, Shape{1, 1, 2}));
        auto v2 = lp2.to_vec();
        float three[3] = {1.f, 0.f, 2.f};
        CHECK(v2[0] == -INFINITY, "excluded token: %g", v2[0]);
        CHECK(std::fabs(v2[1] - log_softmax_row(three, 3)[2]) < 1e-6, "%g", v2[1]);
        Tensor up = Tensor::from_f32({0.f, 1.f}, Shape{1, 1, 2}, dev);
        auto d2 = backward(lp2, up).grad(z2)->to_vec();
        for (float x : d2) CHECK(std::isfinite(x), "a non-finite gradient beside an excluded token");
        CHECK(d2[0] == 0 && d2[1] == 0 && d2[2] == 0 && d2[3] == 0 && d2[5] == 0, "unscored row / excluded entry");
    }
    CHECK(throws([&] { rl::token_log_probs(Tensor::from_f32({0, 0, 0, 0}, Shape{1, 1, 1, 4}, dev), IntTensor::from_data({4}, Shape{1, 1, 1})); }, "out of range"), "token ≥ V");
    CHECK(throws([&] { rl::token_log_probs(Tensor::from_f32({0, 0, 0, 0}, Shape{1, 1, 1, 4}, dev), IntTensor::from_data({0, 1}, Shape{1, 2})); }, "tokens shape"), "tokens shape");
}

// ---- policy_gradient_loss (src/nn/tests/rl.rs:163-207) -----------------------------------------
static void test_policy_gradient() {
    Tensor lp = Tensor::from_f32({-1, -2, -3, -4, -5, -6}, Shape{1, 2, 3}, dev);
    Tensor w = Tensor::from_f32({1, -2}, Shape{1, 2}, dev);
    Tensor m = Tensor::from_f32({1, 1, 0, 0, 1, 0}, Shape{1, 2, 3}, dev);
    auto run = [&](TokenReduction r, const Tensor* mask) { return rl::policy_gradient_loss(lp, w, mask, r).to_vec(); };
    close_all(run(TokenReduction::None, &m), {1, 2, 0, 0, -10, 0}, 0, "pg none");
    close_all(run(TokenReduction::Sum, &m), {-7}, 0, "pg sum");
    close_all(run(TokenReduction::TokenMean, &m), {-7.0 / 3.0}, 1e-7, "pg token mean");
    close_all(run(TokenReduction::PerSequence, &m), {1.5, -10}, 0, "pg per sequence");
    close_all(run(TokenReduction::SequenceMean, &m), {-4.25}, 0, "pg sequence mean");
    close_all(run(TokenReduction::Sum, nullptr), {6.0 - 30.0}, 0, "pg sum unmasked");
    Tensor wt = Tensor::from_f32({1, 1, 1, -2, -2, -2}, Shape{1, 2, 3}, dev);
    close_all(rl::policy_gradient_loss(lp, wt, nullptr, TokenReduction::None).to_vec(), {1, 2, 3, -8, -10, -12}, 0, "pg per-token weights");
    CHECK(throws([&] { rl::policy_gradient_loss(lp, Tensor::from_f32({1, 2, 3}, Shape{1, 3}, dev), nullptr, TokenReduction::Sum); }, "per-sequence weights"), "weights shape");

    // from logits, every reduction, against the f64 host value, and the gradient through both nodes
    Case c = make_case(820, -4.0, 4.0, false);
    std::mt19937_64 g(821);
    std::uniform_real_distribution<double> u(-2, 2);
    std::vector<float> wtok(c.n());
    for (float& x : wtok) x = (float)u(g);
    std::vector<double> host(c.n()), lph(c.n());
    std::vector<std::vector<double>> ys;
    for (size_t i = 0; i < c.n(); i++) {
        ys.push_back(log_softmax_row(&c.logits[i * c.V], c.V));
        lph[i] = ys[i][c.tokens[i]];
        host[i] = c.mask[i] == 1.f ? -(double)wtok[i] * lph[i] : 0.0;
    }
    Tensor mask = Tensor::from_f32(c.mask, c.sh(), dev), wts = Tensor::from_f32(wtok, c.sh(), dev);
    for (TokenReduction r : kReductions) {
        Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev).require_grad();
        Tensor loss = rl::policy_gradient_loss(rl::token_log_probs(z, IntTensor::from_data(c.tokens, c.sh())), wts, &mask, r);
        close_all(loss.to_vec(), reduce_host(host, c.mask, c.S, c.B, c.T, r), 1e-6, "pg from logits");
        if (r != TokenReduction::TokenMean) continue;
        // d/dz of Σ_s token-mean_s: −w_i/count_s · (onehot − softmax) at scored positions, exact 0 elsewhere
        auto d = backward(loss).grad(z)->to_vec();
        for (size_t s = 0; s < c.S; s++) {
            double cnt = 0;
            for (size_t i = s * c.B * c.T; i < (s + 1) * c.B * c.T; i++) cnt += c.mask[i];
            for (size_t i = s * c.B * c.T; i < (s + 1) * c.B * c.T; i++)
                for (size_t v = 0; v < c.V; v++) {
                    double want = c.mask[i] == 1.f ? -(double)wtok[i] / cnt * (((int64_t)v == c.tokens[i] ? 1.0 : 0.0) - std::exp(ys[i][v])) : 0.0;
                    float got = d[i * c.V + v];
                    if (c.mask[i] == 0.f) CHECK(got == 0.f, "unscored position has gradient %g", got);
                    CHECK(std::fabs(got - want) <= 1e-6 * (1 + std::fabs(want)), "pg gradient [%zu,%zu]: %g vs %g", i, v, got, want);
                }
        }
    }
}

// ---- clipped_policy_loss (src/nn/tests/rl.rs:250-332, 676-749) ---------------------------------
static void test_clipped_policy_loss() {
    Case c = make_case(840, -3.0, 3.0, false);
    std::vector<double> lph(c.n());
    for (size_t i = 0; i < c.n(); i++) lph[i] = log_softmax_row(&c.logits[i * c.V], c.V)[c.tokens[i]];
    const double offs[4] = {-0.5, -0.1, 0.05, 0.4};
    std::mt19937_64 g(845);
    std::uniform_real_distribution<double> u(-2, 2);
    std::vector<float> old(c.n()), adv(c.n());
    for (size_t i = 0; i < c.n(); i++) {
        old[i] = (float)(lph[i] + offs[(i * 7 + i / 3) % 4]);
        double a = u(g);
        adv[i] = (float)(std::fabs(a) < 0.1 ? 0.5 : a);
    }
    Tensor mask = Tensor::from_f32(c.mask, c.sh(), dev), to = Tensor::from_f32(old, c.sh(), dev), ta = Tensor::from_f32(adv, c.sh(), dev);
    IntTensor tok = IntTensor::from_data(c.tokens, c.sh());
    for (int dual = 0; dual < 2; dual++) {
        rl::Clip clip = rl::Clip::make(0.2, 0.28);
        if (dual) clip = clip.with_dual(3.0);
        std::vector<double> host(c.n());
        for (size_t i = 0; i < c.n(); i++) {
            double ratio = std::exp(std::min(std::max(lph[i] - (double)old[i], -20.0), 20.0));
            double a = adv[i];
            double l = std::max(-ratio * a, -std::min(std::max(ratio, 0.8), 1.28) * a);
            if (dual && a < 0) l = std::min(l, -3.0 * a);
            host[i] = c.mask[i] == 1.f ? l : 0.0;
        }
        for (TokenReduction r : kReductions) {
            Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev);
            Tensor loss = rl::clipped_policy_loss(rl::token_log_probs(z, tok), to, ta, &mask, clip, r);
            close_all(loss.to_vec(), reduce_host(host, c.mask, c.S, c.B, c.T, r), 2e-6, "clipped_policy_loss");
        }
    }
    // at old = logp the gradient is the policy-gradient loss's with weights = advantages
    {
        Tensor z1 = Tensor::from_f32(c.logits, c.lsh(), dev).require_grad(), z2 = Tensor::from_f32(c.logits, c.lsh(), dev).require_grad();
        Tensor lp1 = rl::token_log_probs(z1, tok), lp2 = rl::token_log_probs(z2, tok);
        Tensor ppo = rl::clipped_policy_loss(lp1, lp1.detach(), ta, &mask, rl::Clip::symmetric(0.2), TokenReduction::SequenceMean);
        Tensor pg = rl::policy_gradient_loss(lp2, ta, &mask, TokenReduction::SequenceMean);
        auto a = backward(ppo).grad(z1)->to_vec(), b = backward(pg).grad(z2)->to_vec();
        std::vector<double> bd(b.begin(), b.end());
        close_all(a, bd, 1e-6, "ppo gradient at ratio 1");
    }
    // garbage at unscored positions never reaches the loss or the gradient
    {
        std::vector<float> lpv = {-1.f, NAN, -2.f, INFINITY}, ov = {-1.1f, 5.f, NAN, -2.f}, av = {1.f, NAN, INFINITY, -1.f}, mv = {1, 0, 0, 0};
        Tensor lp = Tensor::from_f32(lpv, Shape{1, 1, 4}, dev).require_grad();
        Tensor m4 = Tensor::from_f32(mv, Shape{1, 1, 4}, dev);
        Tensor loss = rl::clipped_policy_loss(lp, Tensor::from_f32(ov, Shape{1, 1, 4}, dev), Tensor::from_f32(av, Shape{1, 1, 4}, dev), &m4, rl::Clip::symmetric(0.2), TokenReduction::Sum);
        auto v = loss.to_vec();
        CHECK(std::isfinite(v[0]), "loss %g", v[0]);
        auto d = backward(loss).grad(lp)->to_vec();
        CHECK(std::isfinite(d[0]) && d[1] == 0 && d[2] == 0 && d[3] == 0, "garbage leaked into the gradient");
    }
    CHECK(throws([&] { rl::Clip::make(1.0, 0.2).check(); }, "clip range"), "clip low = 1");
    CHECK(throws([&] { rl::Clip::symmetric(0.2).with_dual(1.0).check(); }, "dual clip"), "dual ≤ 1");
    // clip_fraction: by hand (ratio e^{±0.5} outside [0.8, 1.2] with the advantage's sign making the bound active)
    {
        std::vector<float> lpv = {0.f, 0.f, 0.f, 0.f}, ov = {-0.5f, 0.5f, -0.5f, 0.05f}, av = {1.f, 1.f, -1.f, 1.f};
        Tensor f = rl::clip_fraction(Tensor::from_f32(lpv, Shape{1, 1, 4}, dev), Tensor::from_f32(ov, Shape{1, 1, 4}, dev), Tensor::from_f32(av, Shape{1, 1, 4}, dev), nullptr, rl::Clip::symmetric(0.2));
        close_all(f.to_vec(), {0.25}, 1e-7, "clip_fraction");
    }
}

// ---- categorical_kl / entropy / reference_kl (src/nn/tests/rl.rs:347-423, 773-835) --------------
static void test_kl_entropy() {
    for (int bf = 0; bf < 2; bf++) {
        Case c = make_case(860 + bf, -4.0, 4.0, bf);
        Case r = make_case(870 + bf, -4.0, 4.0, bf);
        std::vector<double> kl(c.n()), en(c.n()), gkl(c.n() * c.V), gen(c.n() * c.V);
        for (size_t i = 0; i < c.n(); i++) {
            auto y = log_softmax_row(&c.logits[i * c.V], c.V), q = log_softmax_row(&r.logits[i * c.V], c.V);
            for (size_t v = 0; v < c.V; v++) {
                kl[i] += std::exp(y[v]) * (y[v] - q[v]);
                en[i] -= std::exp(y[v]) * y[v];
            }
            for (size_t v = 0; v < c.V; v++) {
                gkl[i * c.V + v] = c.mask[i] * std::exp(y[v]) * (y[v] - q[v] - kl[i]);
                gen[i * c.V + v] = -c.mask[i] * std::exp(y[v]) * (y[v] + en[i]);
            }
            kl[i] *= c.mask[i];
            en[i] *= c.mask[i];
        }
        DType dt = bf ? DType::BF16 : DType::F32;
        Tensor mask = Tensor::from_f32(c.mask, c.sh(), dev), zr = Tensor::from_f32(r.logits, c.lsh(), dev, dt);
        for (TokenReduction red : kReductions) {
            Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, dt).require_grad();
            Tensor k = rl::categorical_kl(z, zr, &mask, red), h = rl::categorical_entropy(z, &mask, red);
            close_all(k.to_vec(), reduce_host(kl, c.mask, c.S, c.B, c.T, red), 2e-6, "categorical_kl");
            close_all(h.to_vec(), reduce_host(en, c.mask, c.S, c.B, c.T, red), 2e-6, "categorical_entropy");
            if (red != TokenReduction::Sum) continue;
            close_all(backward(k).grad(z)->to_vec(), gkl, 2e-6, "d categorical_kl");
            close_all(backward(h).grad(z)->to_vec(), gen, 2e-6, "d categorical_entropy");
            // both in one backward: the two nodes add into one d(logits)
            std::vector<double> both(gkl.size());
            for (size_t j = 0; j < both.size(); j++) both[j] = 0.04 * gkl[j] - 0.01 * gen[j];
            close_all(backward(std::vector<Term>{{k, 0.04}, {h, -0.01}}).grad(z)->to_vec(), both, 2e-6, "d (β·kl − c·entropy)");
        }
    }
    // a U8 vocabulary mask and a −1e9 additive mask exclude the same tokens; reference_kl tempers both sides
    {
        Case c = make_case(880, -3.0, 3.0, false), r = make_case(881, -3.0, 3.0, false);
        std::vector<uint8_t> allow(c.V);
        std::vector<float> add(c.V);
        for (size_t v = 0; v < c.V; v++) {
            allow[v] = v % 3 != 1;
            add[v] = allow[v] ? 0.f : -1e9f;
        }
        const double tau = 0.7;
        std::vector<double> kl(c.n());
        for (size_t i = 0; i < c.n(); i++) {
            auto y = log_softmax_row(&c.logits[i * c.V], c.V, tau, allow.data()), q = log_softmax_row(&r.logits[i * c.V], c.V, tau, allow.data());
            for (size_t v = 0; v < c.V; v++)
                if (allow[v]) kl[i] += std::exp(y[v]) * (y[v] - q[v]);
        }
        Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev), zr = Tensor::from_f32(r.logits, c.lsh(), dev);
        Tensor mu = Tensor::from_u8(allow, Shape{1, 1, 1, c.V}, dev), ma = Tensor::from_f32(add, Shape{1, 1, 1, c.V}, dev);
        auto a = rl::reference_kl(z, zr, tau, &mu, nullptr, TokenReduction::None).to_vec();
        auto b = rl::reference_kl(z, zr, tau, &ma, nullptr, TokenReduction::None).to_vec();
        close_all(a, kl, 2e-6, "reference_kl (U8 mask)");
        close_all(b, kl, 2e-6, "reference_kl (−1e9 mask)");
    }
    CHECK(throws([&] { rl::categorical_entropy(Tensor::from_f32({0, 0}, Shape{1, 2}, dev), nullptr, TokenReduction::Sum); }, "[S, B, T, V]"), "rank");
    CHECK(throws([&] { rl::tempered_logits(Tensor::from_f32({0, 0}, Shape{1, 1, 1, 2}, dev), 0.0, nullptr); }, "temperature"), "temperature 0");
}

// ---- kl_estimate (src/nn/tests/rl.rs:438-460, 753-768) -----------------------------------------
static void test_kl_estimate() {
    std::vector<float> lp = {-1.f, -2.f, -0.5f, -3.f}, rf = {-1.5f, -1.f, -0.5f, 30.f};
    Tensor tl = Tensor::from_f32(lp, Shape{1, 2, 2}, dev), tr = Tensor::from_f32(rf, Shape{1, 2, 2}, dev);
    std::vector<double> k1, k2, k3, k3c;
    for (size_t i = 0; i < 4; i++) {
        double d = (double)rf[i] - lp[i];
        k1.push_back(-d);
        k2.push_back(0.5 * d * d);
        k3.push_back(std::exp(d) - d - 1.0);
        double dc = std::min(std::max(d, -20.0), 20.0);
        k3c.push_back(std::exp(dc) - dc - 1.0);
    }
    close_all(rl::kl_estimate(tl, tr, rl::KlEstimator::K1, false, 0, nullptr, TokenReduction::None).to_vec(), k1, 1e-6, "k1");
    close_all(rl::kl_estimate(tl, tr, rl::KlEstimator::K2, false, 0, nullptr, TokenReduction::None).to_vec(), k2, 1e-6, "k2");
    close_all(rl::kl_estimate(tl, tr, rl::KlEstimator::K3, true, rl::KL_DELTA_CLAMP, nullptr, TokenReduction::None).to_vec(), k3c, 1e-6, "k3 clamped");
    // gradient of k3 w.r.t. logp is 1 − e^δ where the clamp is inactive, 0 where it is active
    Tensor leaf = tl.require_grad();
    auto d = backward(rl::kl_estimate(leaf, tr, rl::KlEstimator::K3, true, 20.0, nullptr, TokenReduction::Sum)).grad(leaf)->to_vec();
    close_all(d, {1.0 - std::exp(-0.5), 1.0 - std::exp(1.0), 0.0, 0.0}, 1e-6, "d k3");
    // one logp feeding two losses: the gradients add
    Tensor leaf2 = tl.require_grad();
    Tensor w = Tensor::from_f32({1, 1, 1, 1}, Shape{1, 2, 2}, dev);
    Tensor a = rl::policy_gradient_loss(leaf2, w, nullptr, TokenReduction::Sum), b = rl::kl_estimate(leaf2, tr, rl::KlEstimator::K1, false, 0, nullptr, TokenReduction::Sum);
    close_all(backward(std::vector<Term>{{a, 1.0}, {b, 0.5}}).grad(leaf2)->to_vec(), {-0.5, -0.5, -0.5, -0.5}, 1e-6, "two losses on one logp");
}

// ---- sample_categorical (src/nn/tests/rl.rs:582-637) -------------------------------------------
static void test_sample_categorical() {
    const size_t rows = 64, V = 1000;
    Case c;
    c.S = 1; c.B = 1; c.T = rows;
    std::mt19937_64 g(900);
    std::uniform_real_distribution<double> u(-3, 3), u01(0, 1);
    std::vector<float> z(rows * V), un(rows);
    std::vector<uint8_t> allow(V);
    for (float& x : z) x = (float)u(g);
    for (float& x : un) x = (float)u01(g);
    for (size_t v = 0; v < V; v++) allow[v] = v % 5 != 0;
    Tensor tz = Tensor::from_f32(z, Shape{1, 1, rows, V}, dev), tu = Tensor::from_f32(un, Shape{1, 1, rows}, dev), tm = Tensor::from_u8(allow, Shape{1, 1, 1, V}, dev);
    const double tau = 0.8;
    IntTensor tok = rl::sample_categorical(tz, tau, &tm, &tu);
    CHECK((tok.shape == Shape{1, 1, rows}), "tokens shape");
    size_t boundary = 0;
    for (size_t i = 0; i < rows; i++) {
        auto y = log_softmax_row(&z[i * V], V, tau, allow.data());
        double cdf = 0, target = (double)un[i];
        int64_t want = -1;
        bool near = false;
        for (size_t v = 0; v < V; v++) {
            if (!allow[v]) continue;
            cdf += std::exp(y[v]);
            if (std::fabs(cdf - target) <= 1e-6) near = true;
            if (want < 0 && cdf > target) want = (int64_t)v;
        }
        CHECK(tok.data[i] >= 0 && allow[tok.data[i]], "row %zu drew the excluded token %lld", i, (long long)tok.data[i]);
        if (near) { boundary++; continue; }
        CHECK(tok.data[i] == want, "row %zu: token %lld, inverse CDF gives %lld", i, (long long)tok.data[i], (long long)want);
    }
    CHECK(boundary < rows / 4, "%zu boundary rows", boundary);
    // temperature 0: the first maximum among allowed tokens
    IntTensor gr = rl::sample_categorical(tz, 0.0, &tm, nullptr);
    for (size_t i = 0; i < rows; i++) {
        size_t best = 1;
        for (size_t v = 0; v < V; v++)
            if (allow[v] && z[i * V + v] > z[i * V + best]) best = v;
        CHECK(gr.data[i] == (int64_t)best, "greedy row %zu", i);
    }
    // a position with no allowed token is refused
    std::vector<float> none(2 * 4, -INFINITY);
    none[0] = 0.f;
    CHECK(throws([&] { rl::sample_categorical(Tensor::from_f32(none, Shape{1, 1, 2, 4}, dev), 1.0, nullptr, &tu); }, "one uniform per position"), "uniform count");
    Tensor u2 = Tensor::from_f32({0.3f, 0.6f}, Shape{1, 1, 2}, dev);
    CHECK(throws([&] { rl::sample_categorical(Tensor::from_f32(none, Shape{1, 1, 2, 4}, dev), 1.0, nullptr, &u2); }, "position 1 has no allowed token"), "all-excluded row");
    CHECK(throws([&] { rl::sample_categorical(tz, -1.0, nullptr, &tu); }, "temperature"), "negative temperature");
}

// ---- sample_categorical with the reference's own noise (src/nn/rl.rs:490-529) -------------------
// Host restatement for the check: ChaCha20 (RFC 8439 block function, 64-bit counter, as
// rand_chacha's ChaCha20Rng), one u64 per logit, noise in f64, first maximum in f32.
struct HostChaCha {
    uint32_t key[8];
    uint64_t counter = 0;
    uint32_t buf[16];
    int idx = 16;
    static uint32_t rotl(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }
    static void qr(uint32_t* s, int a, int b, int c, int d) {
        s[a] += s[b]; s[d] ^= s[a]; s[d] = rotl(s[d], 16);
        s[c] += s[d]; s[b] ^= s[c]; s[b] = rotl(s[b], 12);
        s[a] += s[b]; s[d] ^= s[a]; s[d] = rotl(s[d], 8);
        s[c] += s[d]; s[b] ^= s[c]; s[b] = rotl(s[b], 7);
    }
    explicit HostChaCha(const uint8_t seed[32]) {
        for (int i = 0; i < 8; i++) key[i] = (uint32_t)seed[4 * i] | (uint32_t)seed[4 * i + 1] << 8 | (uint32_t)seed[4 * i + 2] << 16 | (uint32_t)seed[4 * i + 3] << 24;
    }
    uint32_t next_u32() {
        if (idx >= 16) {
            uint32_t in[16] = {0x61707865, 0x3320646e, 0x79622d32, 0x6b206574};
            for (int i = 0; i < 8; i++) in[4 + i] = key[i];
            in[12] = (uint32_t)counter; in[13] = (uint32_t)(counter >> 32); in[14] = in[15] = 0;
            uint32_t s[16];
            std::memcpy(s, in, sizeof s);
            for (int r = 0; r < 10; r++) {
                qr(s, 0, 4, 8, 12); qr(s, 1, 5, 9, 13); qr(s, 2, 6, 10, 14); qr(s, 3, 7, 11, 15);
                qr(s, 0, 5, 10, 15); qr(s, 1, 6, 11, 12); qr(s, 2, 7, 8, 13); qr(s, 3, 4, 9, 14);
            }
            for (int i = 0; i < 16; i++) buf[i] = s[i] + in[i];
            counter++;
            idx = 0;
        }
        return buf[idx++];
    }
    uint64_t next_u64() {
        uint64_t lo = next_u32(), hi = next_u32();
        return hi << 32 | lo;
    }
};

static void test_sample_categorical_reference() {
    using rl::ChaChaStream;
    const size_t rows = 24, V = 1000;
    std::mt19937_64 g(930);
    std::uniform_real_distribution<double> u(-3, 3);
    std::vector<float> z(rows * V), add(V);
    for (float& x : z) x = (float)u(g);
    for (size_t v = 0; v < V; v++) add[v] = v % 7 == 3 ? -INFINITY : 0.f;
    Tensor tz = Tensor::from_f32(z, Shape{1, 2, rows / 2, V}, dev), tm = Tensor::from_f32(add, Shape{1, 1, 1, V}, dev);
    ChaChaStream rng;
    for (int i = 0; i < 32; i++) rng.seed[i] = (uint8_t)(37 * i + 11);
    const float tau = 0.7f;
    IntTensor first = rl::sample_categorical(tz, tau, &tm, rng);
    CHECK(rng.words == 2 * rows * V, "the generator advanced by %llu words", (unsigned long long)rng.words);
    IntTensor second = rl::sample_categorical(tz, tau, &tm, rng);  // continues the same stream
    HostChaCha h(rng.seed);
    for (int pass = 0; pass < 2; pass++) {
        const IntTensor& got = pass ? second : first;
        for (size_t r = 0; r < rows; r++) {
            float best = -INFINITY;
            int64_t bi = -1;
            for (size_t v = 0; v < V; v++) {
                const uint64_t k = h.next_u64() >> 11;
                const double uu = ((double)k + 0.5) / 9007199254740992.0;
                const float gn = (float)(-std::log(-std::log(uu)));
                const float y = (z[r * V + v] / tau + add[v]) + gn;
                if (y > best) { best = y; bi = (int64_t)v; }
            }
            CHECK(got.data[r] == bi, "pass %d row %zu: token %lld, the reference sampler gives %lld", pass, r, (long long)got.data[r], (long long)bi);
            CHECK(got.data[r] % 7 != 3, "an excluded token was drawn");
        }
    }
    ChaChaStream again = rng;
    again.words = 0;
    CHECK(rl::sample_categorical(tz, tau, &tm, again).data == first.data, "the same generator state gives the same tokens");
    // temperature 0 draws nothing
    ChaChaStream still = rng;
    rl::sample_categorical(tz, 0.0, &tm, still);
    CHECK(still.words == rng.words, "greedy sampling consumed the generator");
}

// ---- group_advantages (src/nn/tests/rl.rs:550-575, 644-653) ------------------------------------
static void test_group_advantages() {
    auto a = rl::group_advantages({1, 2, 3, 5, 5, 5}, 3, rl::GroupNorm::MeanOnly());
    CHECK((a == std::vector<double>{-1, 0, 1, 0, 0, 0}), "mean only");
    auto b = rl::group_advantages({1, 2, 3, 4}, 2, rl::GroupNorm::Std(0.0, true));
    const double s = std::sqrt(0.5);
    CHECK(std::fabs(b[0] + 0.5 / s) < 1e-15 && std::fabs(b[3] - 0.5 / s) < 1e-15, "std");
    auto z = rl::group_advantages({0.1, 0.1, 0.1}, 3, rl::GroupNorm::Std(0.0, true));
    CHECK((z == std::vector<double>{0, 0, 0}), "equal rewards");
    CHECK(throws([] { rl::group_advantages({1, 2, 3}, 2, rl::GroupNorm::MeanOnly()); }, "groups of n"), "ragged");
    CHECK(throws([] { rl::group_advantages({1, 2}, 1, rl::GroupNorm::Std(0.0, true)); }, "at least 2"), "n = 1 unbiased");
    // group_advantages_tensor on the device: the host function's values rounded to f32 once
    const std::vector<float> r32 = {1, 0, 0, 1, 0.25f, 0.5f, 4, 8, 3, 3, 3, 3};
    const std::vector<double> r64(r32.begin(), r32.end());
    for (auto norm : {rl::GroupNorm::MeanOnly(), rl::GroupNorm::Std(0.0, true), rl::GroupNorm::Std(1e-6, false)}) {
        auto want = rl::group_advantages(r64, 4, norm);
        auto got = rl::group_advantages_tensor(Tensor::from_f32(r32, {3, 4}, dev), norm).to_vec();
        bool same = true;
        for (size_t i = 0; i < want.size(); i++) same = same && got[i] == (float)want[i];
        CHECK(same, "group_advantages_tensor equals the host function");
    }
    CHECK(throws([] { rl::group_advantages_tensor(Tensor::from_f32({1, 2}, {2, 1}, dev), rl::GroupNorm::Std(0.0, true)); }, "at least 2"), "tensor n = 1 unbiased");
}

// ---- Decoder::head fused with token_log_probs / categorical_entropy (tcgen05) -------------------------
static void test_head_token_log_probs() {
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, 0);
    if (prop.major != 10) {
        std::printf("    (skipped: needs compute capability 10.x, this device is %d.%d)\n", prop.major, prop.minor);
        return;
    }
    const size_t S = 2, B = 3, T = 50, d = 72, V = 776;  // 300 rows: CTA pairs, a ragged last block, a ragged last tile
    std::mt19937 gen(7);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> x(S * B * T * d), w(d * V);
    for (auto& v : x) v = through_bf16(nd(gen));
    for (auto& v : w) v = through_bf16(nd(gen) * 0.35f);
    std::vector<int64_t> tok(S * B * T);
    for (size_t i = 0; i < tok.size(); i++) tok[i] = (int64_t)(gen() % V);
    Tensor hx = Tensor::from_f32(x, {S, B, T, d}, dev, DType::BF16), hw = Tensor::from_f32(w, {d, V}, dev, DType::BF16);
    IntTensor it = IntTensor::from_data(tok, Shape{S, B, T});
    Tensor ent;
    const std::vector<float> lp = rl::head_token_log_probs(hx, hw, it, &ent).to_vec(), en = ent.to_vec();
    // f64 on the host: logits = x · w, then log-softmax and entropy
    std::vector<double> want_lp(tok.size()), want_en(tok.size());
    for (size_t r = 0; r < tok.size(); r++) {
        std::vector<double> z(V, 0.0);
        for (size_t k = 0; k < d; k++)
            for (size_t v = 0; v < V; v++) z[v] += (double)x[r * d + k] * (double)w[k * V + v];
        double m = z[0];
        for (double v : z) m = std::max(m, v);
        double Z = 0.0;
        for (double v : z) Z += std::exp(v - m);
        const double lse = m + std::log(Z);
        double h = 0.0;
        for (double v : z) h -= std::exp(v - lse) * (v - lse);
        want_lp[r] = z[tok[r]] - lse;
        want_en[r] = h;
    }
    close_all(lp, want_lp, 2e-5, "head_token_log_probs");
    close_all(en, want_en, 2e-5, "head entropy");
    CHECK(throws([&] { rl::head_token_log_probs(Tensor::from_f32(x, {S, B, T, d}, dev), hw, it); }, "BF16"), "f32 hidden states are refused");
}

// ---- Decoder::head fused with sample_categorical (inverse CDF), masks included ------------------------------
static void test_head_sample_categorical() {
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, 0);
    if (prop.major != 10) {
        std::printf("    (skipped: needs compute capability 10.x, this device is %d.%d)\n", prop.major, prop.minor);
        return;
    }
    const size_t S = 2, B = 2, T = 40, d = 64, V = 512, rows = S * B * T;
    std::mt19937 gen(11);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_real_distribution<float> ud(0.f, 1.f);
    std::vector<float> x(rows * d), w(d * V), u(rows);
    for (auto& v : x) v = through_bf16(nd(gen));
    for (auto& v : w) v = through_bf16(nd(gen) * 0.35f);
    for (auto& v : u) v = std::min(ud(gen), 0.99999994f);
    std::vector<uint8_t> mask(rows * V);
    for (size_t i = 0; i < mask.size(); i++) mask[i] = (gen() % 4) == 0;
    for (size_t r = 0; r < rows; r++) mask[r * V + 5] = 1;
    Tensor hx = Tensor::from_f32(x, {S, B, T, d}, dev, DType::BF16), hw = Tensor::from_f32(w, {d, V}, dev, DType::BF16);
    Tensor hu = Tensor::from_f32(u, {S, B, T}, dev), hm = Tensor::from_u8(mask, {S, B, T, V}, dev);
    Tensor lpt, ent;
    const IntTensor tok = rl::head_sample_categorical(hx, hw, hu, &hm, &lpt, &ent);
    const std::vector<float> lp = lpt.to_vec(), en = ent.to_vec();
    CHECK(tok.shape == (Shape{S, B, T}), "token shape");
    // f64 on the host: masked logits, the inverse CDF's interval of the drawn token must hold u (up to the f32 spread of a logit)
    size_t outside = 0;
    std::vector<double> want_lp(rows), want_en(rows);
    for (size_t r = 0; r < rows; r++) {
        std::vector<double> z(V, 0.0);
        for (size_t k = 0; k < d; k++)
            for (size_t v = 0; v < V; v++) z[v] += (double)x[r * d + k] * (double)w[k * V + v];
        double m = -1e300;
        for (size_t v = 0; v < V; v++)
            if (mask[r * V + v]) m = std::max(m, z[v]);
        double Z = 0.0;
        for (size_t v = 0; v < V; v++)
            if (mask[r * V + v]) Z += std::exp(z[v] - m);
        const double lse = m + std::log(Z);
        double h = 0.0, lo = 0.0;
        const int64_t t = tok.data[r];
        CHECK(t >= 0 && (size_t)t < V && mask[r * V + t], "row %zu: token %lld is not an allowed one", r, (long long)t);
        for (size_t v = 0; v < V; v++) {
            if (!mask[r * V + v]) continue;
            const double pv = std::exp(z[v] - lse);
            h -= pv * (z[v] - lse);
            if ((int64_t)v < t) lo += pv;
        }
        const double hi = lo + std::exp(z[t] - lse);
        if (!((double)u[r] >= lo - 1e-4 && (double)u[r] <= hi + 1e-4)) outside++;
        want_lp[r] = z[t] - lse;
        want_en[r] = h;
    }
    CHECK(outside == 0, "%zu drawn tokens whose CDF interval does not hold the uniform", outside);
    close_all(lp, want_lp, 1e-4, "head_sample_categorical log-probs");
    close_all(en, want_en, 2e-5, "head_sample_categorical entropy");
    // temperature 0: the first maximum among the allowed tokens (f64 logits; an f32 near-tie may pick a neighbour of equal value only)
    const IntTensor top = rl::head_sample_categorical(hx, hw, hu, &hm, nullptr, nullptr, 0.0);
    size_t off_max = 0;
    for (size_t r = 0; r < rows; r++) {
        double best = -1e300, mine = 0.0;
        for (size_t v = 0; v < V; v++) {
            if (!mask[r * V + v]) continue;
            double z = 0.0;
            for (size_t k = 0; k < d; k++) z += (double)x[r * d + k] * (double)w[k * V + v];
            best = std::max(best, z);
            if ((int64_t)v == top.data[r]) mine = z;
        }
        if (!(top.data[r] >= 0 && mask[r * V + top.data[r]] && best - mine <= 1e-4)) off_max++;
    }
    CHECK(off_max == 0, "%zu greedy tokens are not a maximum of the allowed logits", off_max);
    std::vector<uint8_t> none(mask);
    for (size_t v = 0; v < V; v++) none[7 * V + v] = 0;
    Tensor hn = Tensor::from_u8(none, {S, B, T, V}, dev);
    CHECK(throws([&] { rl::head_sample_categorical(hx, hw, hu, &hn); }, "position 7 has no allowed token"), "a position with nothing allowed is refused by name");
}

// ---- check_scored_finite (src/nn/tests/rl.rs:837-855) -------------------------------------------
static void test_check_scored_finite() {
    const float ninf = -std::numeric_limits<float>::infinity();
    Tensor lp = Tensor::from_f32({-1.0f, ninf, -2.0f}, {1, 1, 3}, dev);
    const std::string e = rl::check_scored_finite("test", lp, nullptr);
    CHECK(e.find("position 1") != std::string::npos && e == "test: the scored log-probability at flat position 1 is -inf (not finite)", "%s", e.c_str());
    Tensor m = Tensor::from_f32({1.0f, 0.0f, 1.0f}, {1, 1, 3}, dev);
    CHECK(rl::check_scored_finite("test", lp, &m).empty(), "a -inf at a masked position passes");
    CHECK(rl::check_scored_finite("test", Tensor::from_f32({-1.0f, -3.0f, -2.0f}, {1, 1, 3}, dev), nullptr).empty(), "finite values pass");
    Tensor nan = Tensor::from_f32({-1.0f, -2.0f, std::nanf("")}, {1, 1, 3}, dev);
    CHECK(rl::check_scored_finite("x", nan, nullptr) == "x: the scored log-probability at flat position 2 is NaN (not finite)", "NaN is named");
#ifndef NDEBUG
    // debug builds refuse a scored log-probability of -inf in the losses
    Tensor two = Tensor::from_f32({-1.0f, ninf}, {1, 1, 2}, dev);
    Tensor w = Tensor::from_f32({1.0f}, {1, 1}, dev);
    CHECK(throws([&] { rl::policy_gradient_loss(two, w, nullptr, TokenReduction::Sum); }, "not finite"), "policy_gradient_loss refuses");
    Tensor old = Tensor::from_f32({-1.0f, -1.0f}, {1, 1, 2}, dev);
    CHECK(throws([&] { rl::clipped_policy_loss(old, two, w, nullptr, rl::Clip::symmetric(0.2), TokenReduction::Sum); }, "clipped_policy_loss (old log-probabilities)"), "old log-probs checked");
    CHECK(throws([&] { rl::kl_estimate(old, two, rl::KlEstimator::K3, false, 0.0, nullptr, TokenReduction::Sum); }, "kl_estimate (reference log-probabilities)"), "reference log-probs checked");
    Tensor skip = Tensor::from_f32({1.0f, 0.0f}, {1, 1, 2}, dev);
    (void)rl::policy_gradient_loss(two, w, &skip, TokenReduction::Sum);  // unscored: passes
#endif
}

// ---- bit-packed vocabulary masks: the same results as the byte mask, bit for bit --------------------
static void test_bit_masks() {
    const size_t S = 2, B = 3, T = 4, V = 200, rows = S * B * T, words = (V + 31) / 32;
    std::vector<float> x(rows * V), u(rows);
    std::vector<uint8_t> m(rows * V);
    std::vector<int32_t> bits(rows * words, 0);
    uint32_t st = 12345u;
    auto rnd = [&]() { st = st * 1664525u + 1013904223u; return (float)(st >> 8) / 16777216.0f; };
    for (size_t i = 0; i < x.size(); i++) { x[i] = 6.f * rnd() - 3.f; m[i] = rnd() < 0.3f ? 1 : 0; }
    for (size_t r = 0; r < rows; r++) {
        m[r * V + 7] = 1;
        u[r] = rnd();
        for (size_t v = 0; v < V; v++)
            if (m[r * V + v]) bits[r * words + v / 32] |= (int32_t)(1u << (v % 32));
    }
    Tensor tx = Tensor::from_f32(x, {S, B, T, V}, dev).require_grad();
    Tensor tm = Tensor::from_u8(m, {S, B, T, V}, dev);
    Tensor tb = Tensor::empty({S, B, T, words}, noetic::DType::I32, dev);
    noetic::cu(cudaMemcpy(tb.ptr(), bits.data(), bits.size() * 4, cudaMemcpyHostToDevice), "upload bits");
    Tensor tu = Tensor::from_f32(u, {S, B, T}, dev);
    IntTensor ta = rl::sample_categorical(tx, 1.0, &tm, &tu), tc = rl::sample_categorical(tx, 1.0, &tb, &tu);
    CHECK(ta.data == tc.data, "bit mask: sampled tokens");
    Tensor la = rl::token_log_probs(rl::tempered_logits(tx, 1.0, &tm), ta), lb = rl::token_log_probs(rl::tempered_logits(tx, 1.0, &tb), ta);
    CHECK(la.to_vec() == lb.to_vec(), "bit mask: log-probs");
    Tensor ea = rl::categorical_entropy(rl::tempered_logits(tx, 1.0, &tm), nullptr, rl::TokenReduction::TokenMean);
    Tensor eb = rl::categorical_entropy(rl::tempered_logits(tx, 1.0, &tb), nullptr, rl::TokenReduction::TokenMean);
    CHECK(ea.to_vec() == eb.to_vec(), "bit mask: entropy");
    // entropy token-mean is [S]: weight every seed by 1
    Tensor up = Tensor::from_f32({1.f, 1.f}, {S}, dev);
    auto ga = backward(ea, up).grad(tx)->to_vec(), gb = backward(eb, up).grad(tx)->to_vec();
    CHECK(ga == gb, "bit mask: d(logits)");
}

// ---- lane operations (src/tensor/tests/standard.rs:8-24, 101-109; checks.rs:103-114) -------------
static void test_lane_ops() {
    const float inf = INFINITY, nan = NAN;
    auto lse = noetic::lane::logsumexp(Tensor::from_f32({1000, 1000, -inf, 0, -inf, -inf, -inf, -inf, 1, inf, 0, 2, 0.5f, nan, 1, 3}, {4, 4}, dev)).to_vec();
    CHECK(std::fabs(lse[0] - (1000.0f + 0.6931472f)) < 1e-3f && lse[1] == -inf && lse[2] == inf && std::isnan(lse[3]), "logsumexp at infinities");
    auto am = noetic::lane::argmax(Tensor::from_f32({1, nan, 5, 2, nan, 3, 9, 0, 4, nan, nan, 1, 1, 7, 7, 2}, {4, 4}, dev));
    std::vector<int32_t> idx(4);
    noetic::cu(cudaMemcpy(idx.data(), am.first.ptr(), 16, cudaMemcpyDeviceToHost), "download");
    CHECK((idx == std::vector<int32_t>{1, 0, 1, 1}), "argmax: the first NaN is the maximum, ties take the first");
    auto sm = noetic::lane::softmax(Tensor::from_f32({0.5f, nan, -1, 2, -inf, -inf, -inf, -inf, 1, -inf, 3, -inf}, {3, 4}, dev)).to_vec();
    bool nans = true;
    for (int i = 0; i < 8; i++) nans = nans && std::isnan(sm[i]);
    CHECK(nans && sm[9] == 0.f && std::fabs(sm[8] + sm[10] - 1.f) < 1e-6f, "softmax of NaN / all -inf / partly masked rows");
    std::vector<float> x(3 * 37);
    for (size_t i = 0; i < x.size(); i++) x[i] = std::sin((float)i) * 4.f;
    auto ls = noetic::lane::log_softmax(Tensor::from_f32(x, {3, 37}, dev)).to_vec();
    auto su = noetic::lane::sum_last(Tensor::from_f32(x, {3, 37}, dev)).to_vec();
    for (int r = 0; r < 3; r++) {
        double m = -1e30, z = 0, s = 0;
        for (int j = 0; j < 37; j++) m = std::max(m, (double)x[r * 37 + j]);
        for (int j = 0; j < 37; j++) { z += std::exp(x[r * 37 + j] - m); s += x[r * 37 + j]; }
        bool ok = std::fabs(su[r] - s) < 1e-4;
        for (int j = 0; j < 37; j++) ok = ok && std::fabs(ls[r * 37 + j] - (x[r * 37 + j] - m - std::log(z))) < 1e-5;
        CHECK(ok, "log_softmax and sum_last against f64");
    }
}

// ---- a PPO step end to end: clipped loss + β·reference_kl − c·entropy, one backward -------------
static void test_ppo_step() {
    Case c = make_case(910, -3.0, 3.0, true, 515), r = make_case(911, -3.0, 3.0, true, 515);
    IntTensor tok = IntTensor::from_data(c.tokens, c.sh());
    Tensor mask = Tensor::from_f32(c.mask, c.sh(), dev);
    Tensor zr = Tensor::from_f32(r.logits, c.lsh(), dev, DType::BF16);
    std::vector<float> adv(c.n());
    for (size_t i = 0; i < c.n(); i++) adv[i] = (i % 3 == 0) ? -1.f : 0.75f;
    Tensor ta = Tensor::from_f32(adv, c.sh(), dev);
    Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, DType::BF16).require_grad();
    Tensor lp = rl::token_log_probs(z, tok);
    Tensor ppo = rl::clipped_policy_loss(lp, lp.detach(), ta, &mask, rl::Clip::symmetric(0.2), TokenReduction::Sum);
    Tensor kl = rl::categorical_kl(z, zr, &mask, TokenReduction::Sum);
    Tensor en = rl::categorical_entropy(z, &mask, TokenReduction::Sum);
    uint64_t before = nrl_launch_count();
    auto d = backward(std::vector<Term>{{ppo, 1.0}, {kl, 0.04}, {en, -0.01}}).grad(z)->to_vec();
    uint64_t launches = nrl_launch_count() - before;
    std::vector<double> want(c.n() * c.V);
    for (size_t i = 0; i < c.n(); i++) {
        auto y = log_softmax_row(&c.logits[i * c.V], c.V), q = log_softmax_row(&r.logits[i * c.V], c.V);
        double k = 0, h = 0;
        for (size_t v = 0; v < c.V; v++) {
            k += std::exp(y[v]) * (y[v] - q[v]);
            h -= std::exp(y[v]) * y[v];
        }
        for (size_t v = 0; v < c.V; v++) {
            double p = std::exp(y[v]);
            double g = -(double)adv[i] * (((int64_t)v == c.tokens[i] ? 1.0 : 0.0) - p) + 0.04 * p * (y[v] - q[v] - k) + 0.01 * p * (y[v] + h);
            want[i * c.V + v] = c.mask[i] * g;
        }
    }
    close_all(d, want, 3e-6, "d(ppo + β·kl − c·entropy)");
    std::printf("  PPO step backward: %llu kernel launches for 3 loss terms over %zu rows\n", (unsigned long long)launches, c.n());
}

// ---- nn::loss cross-entropy family (src/nn/tests/naive.rs:152-170, components.rs:534-588) -------
static void test_loss_family() {
    namespace ls = noetic::nn::loss;
    for (int bf = 0; bf < 2; bf++) {
        Case c = make_case(940 + bf, -3.0, 3.0, bf, bf ? 1000 : 5);
        const size_t N = c.B * c.T;
        std::vector<int64_t> tg = c.tokens, tg_ign = c.tokens;
        tg_ign[1] = -100;
        tg_ign[7] = -100;
        std::vector<std::vector<double>> ys;
        for (size_t i = 0; i < c.n(); i++) ys.push_back(log_softmax_row(&c.logits[i * c.V], c.V));
        auto host = [&](const std::vector<int64_t>& t, bool masked, bool ignore, double eps, std::vector<double>* grad) {
            std::vector<double> out(c.S);
            if (grad) grad->assign(c.n() * c.V, 0.0);
            for (size_t s = 0; s < c.S; s++) {
                double sum = 0, cnt = 0;
                for (size_t i = s * N; i < (s + 1) * N; i++) {
                    double keep = masked ? c.mask[i] : 1.0;
                    if (ignore && t[i] == -100) keep = 0.0;
                    cnt += keep;
                }
                for (size_t i = s * N; i < (s + 1) * N; i++) {
                    double keep = masked ? c.mask[i] : 1.0;
                    int64_t ti = t[i];
                    if (ignore && ti == -100) { keep = 0.0; ti = 0; }
                    double mean = 0;
                    for (size_t v = 0; v < c.V; v++) mean += ys[i][v];
                    mean /= (double)c.V;
                    sum += keep * ((1 - eps) * -ys[i][ti] + eps * -mean);
                    if (grad)
                        for (size_t v = 0; v < c.V; v++)
                            (*grad)[i * c.V + v] = keep / std::max(cnt, 1.0) * (std::exp(ys[i][v]) - (1 - eps) * ((int64_t)v == ti ? 1.0 : 0.0) - eps / (double)c.V);
                }
                out[s] = sum / std::max(cnt, 1.0);
            }
            return out;
        };
        DType dt = bf ? DType::BF16 : DType::F32;
        Tensor mask = Tensor::from_f32(c.mask, c.sh(), dev);
        IntTensor t0 = IntTensor::from_data(tg, c.sh()), t1 = IntTensor::from_data(tg_ign, c.sh());
        std::vector<double> gw;
        {
            Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, dt).require_grad();
            Tensor l = ls::cross_entropy(z, t0);
            close_all(l.to_vec(), host(tg, false, false, 0.0, &gw), 2e-6, "cross_entropy");
            close_all(backward(l).grad(z)->to_vec(), gw, 2e-6, "d cross_entropy");
            std::vector<double> nl;
            for (size_t i = 0; i < c.n(); i++) nl.push_back(-ys[i][tg[i]]);
            Tensor per = ls::nll(z, t0);
            CHECK((per.shape() == Shape{c.S, N}), "nll shape");
            close_all(per.to_vec(), nl, 2e-6, "nll");
        }
        {
            Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, dt).require_grad();
            Tensor l = ls::masked_cross_entropy(z, t0, mask);
            close_all(l.to_vec(), host(tg, true, false, 0.0, &gw), 2e-6, "masked_cross_entropy");
            auto d = backward(l).grad(z)->to_vec();
            close_all(d, gw, 2e-6, "d masked_cross_entropy");
            for (size_t i = 0; i < c.n(); i++)
                if (c.mask[i] == 0.f)
                    for (size_t v = 0; v < c.V; v++) CHECK(d[i * c.V + v] == 0.f, "unscored position has a gradient");
            // default options are the plain losses, to the bit
            auto a = ls::cross_entropy_with(z, t0, &mask, ls::CeOptions()).to_vec(), b = l.to_vec();
            CHECK(std::memcmp(a.data(), b.data(), a.size() * 4) == 0, "default options differ from masked_cross_entropy");
        }
        {
            Tensor z = Tensor::from_f32(c.logits, c.lsh(), dev, dt).require_grad();
            Tensor l = ls::cross_entropy_with(z, t1, &mask, ls::CeOptions::ignore(-100).with_smoothing(0.1));
            close_all(l.to_vec(), host(tg_ign, true, true, 0.1, &gw), 2e-6, "cross_entropy_with");
            close_all(backward(l).grad(z)->to_vec(), gw, 2e-6, "d cross_entropy_with");
            CHECK(throws([&] { ls::cross_entropy(z, t1); }, "one_hot: -100 is outside"), "-100 without ignore_index");
            CHECK(throws([&] { ls::cross_entropy_with(z, t0, nullptr, ls::CeOptions().with_smoothing(1.5)); }, "label smoothing"), "smoothing 1.5");
        }
        // kl_div: value, KL(a, a) = 0, and both gradients
        {
            Case r = make_case(950 + bf, -2.0, 2.0, bf, c.V);
            Tensor q = Tensor::from_f32(c.logits, c.lsh(), dev, dt).require_grad(), p = Tensor::from_f32(r.logits, c.lsh(), dev, dt).require_grad();
            Tensor k = ls::kl_div(q, p);
            std::vector<double> want(c.S, 0.0), gq(c.n() * c.V), gp(c.n() * c.V);
            for (size_t i = 0; i < c.n(); i++) {
                auto lp = log_softmax_row(&r.logits[i * c.V], c.V);
                double per = 0;
                for (size_t v = 0; v < c.V; v++) per += std::exp(lp[v]) * (lp[v] - ys[i][v]);
                want[i / N] += per / (double)N;
                for (size_t v = 0; v < c.V; v++) {
                    gq[i * c.V + v] = (std::exp(ys[i][v]) - std::exp(lp[v])) / (double)N;
                    gp[i * c.V + v] = std::exp(lp[v]) * (lp[v] - ys[i][v] - per) / (double)N;
                }
            }
            close_all(k.to_vec(), want, 2e-6, "kl_div");
            Gradients g = backward(k);
            close_all(g.grad(q)->to_vec(), gq, 2e-6, "d kl_div / d pred");
            close_all(g.grad(p)->to_vec(), gp, 2e-6, "d kl_div / d target");
            for (float x : ls::kl_div(q, q.detach()).to_vec()) CHECK(std::fabs(x) < 1e-6, "KL(a, a) = %g", x);
            // a fixed teacher: only the prediction gets a gradient
            Tensor k2 = ls::kl_div(q, p.detach());
            Gradients g2 = backward(k2);
            close_all(g2.grad(q)->to_vec(), gq, 2e-6, "d kl_div / d pred, detached target");
        }
    }
}

int main() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        std::printf("no CUDA device: this program tests the GPU path and has nothing to fall back to\n");
        return 2;
    }
    std::printf("library: %s\n", nrl_key());
    struct { const char* name; void (*fn)(); } tests[] = {
        {"token_log_probs", test_token_log_probs}, {"policy_gradient_loss", test_policy_gradient},
        {"clipped_policy_loss", test_clipped_policy_loss}, {"categorical_kl / entropy / reference_kl", test_kl_entropy},
        {"kl_estimate", test_kl_estimate}, {"sample_categorical", test_sample_categorical},
        {"sample_categorical (reference noise)", test_sample_categorical_reference},
        {"group_advantages", test_group_advantages}, {"check_scored_finite", test_check_scored_finite}, {"head + token_log_probs (readout-fused)", test_head_token_log_probs}, {"head + sample_categorical (readout-fused)", test_head_sample_categorical}, {"lane operations", test_lane_ops}, {"bit-packed masks", test_bit_masks}, {"ppo step", test_ppo_step},
        {"nn::loss cross-entropy family", test_loss_family},
    };
    for (auto& t : tests) {
        try {
            t.fn();
        } catch (const std::exception& e) {
            std::printf("FAILED %s: exception: %s\n", t.name, e.what());
            return 1;
        }
        std::printf("ok  %s\n", t.name);
    }
    std::printf("all passed: %d checks\n", g_checks);
    return 0;
}
