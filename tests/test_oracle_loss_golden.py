"""Pins the CPU oracle's cross-entropy family (oracle/loss.hpp) against the naive f64 formulas,
identities and tolerances of the reference's own tests of `nn::loss` (src/nn/tests/naive.rs,
src/nn/tests/components.rs, src/nn/tests/rl.rs; each test names the lines it restates). The
reference draws its cases from ChaCha8Rng; here numpy-seeded data of the same shapes and ranges
is used and the comparisons are the reference's. CPU only."""
import numpy as np

INF = float("inf")


def close(got, want, tol):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.where(got == want, 0.0, np.abs(got - want) / (1.0 + np.abs(want)))
    assert np.all(err <= tol), f"max error {np.nanmax(err):.3e} > {tol}"


def log_softmax(x):
    m = x.max(-1, keepdims=True)
    return x - m - np.log(np.exp(x - m).sum(-1, keepdims=True))


def test_losses_match_naive(oracle):
    # src/nn/tests/naive.rs:152-170
    S, B, T, V = 3, 2, 4, 5
    g = np.random.default_rng(40)
    logits = g.uniform(-3, 3, (S, B, T, V))
    targets = g.integers(0, V, (S, B, T))
    mask = (g.uniform(0, 1, (S, B, T)) < 0.5).astype(np.float64)
    mask[2] = 0.0  # seed 2 scores nothing
    lp = log_softmax(logits)
    nll = -np.take_along_axis(lp, targets[..., None], -1)[..., 0].reshape(S, B * T)
    sh = (S, B, T, V)
    close(oracle.rl_eval(oracle.OP_NLL, sh, dtype=oracle.F64, logits=logits, tokens=targets), nll.ravel(), 1e-12)
    close(oracle.rl_eval(oracle.OP_CE, sh, dtype=oracle.F64, logits=logits, tokens=targets), nll.mean(1), 1e-12)
    m = mask.reshape(S, B * T)
    got = oracle.rl_eval(oracle.OP_MASKED_CE, sh, dtype=oracle.F64, logits=logits, tokens=targets, mask=mask)
    close(got, (nll * m).sum(1) / np.maximum(m.sum(1), 1.0), 1e-12)
    assert got[2] == 0.0
    # f32 engine within the reference's f32 tolerance of the same values
    close(oracle.rl_eval(oracle.OP_CE, sh, dtype=oracle.F32, logits=logits, tokens=targets), nll.mean(1), 1e-6)


def test_kl_div_matches_naive_and_its_gradients(oracle):
    # src/nn/tests/components.rs:536-548: value against the naive sum, KL >= 0, KL(a, a) = 0, and
    # the gradient with respect to the prediction (the reference checks it by finite differences;
    # the closed form is (Q − P)/n per position)
    S, B, T, V = 2, 2, 3, 5
    n = B * T
    g = np.random.default_rng(70)
    a, c = g.uniform(-2, 2, (S, B, T, V)), g.uniform(-2, 2, (S, B, T, V))
    lq, lp = log_softmax(a), log_softmax(c)
    want = (np.exp(lp) * (lp - lq)).sum(-1).reshape(S, n).mean(1)
    sh = (S, B, T, V)
    kl, gq, gp = oracle.rl_eval(oracle.OP_KL_DIV, sh, dtype=oracle.F64, logits=a, ref_logits=c, upstream=np.ones(S), grad_ref=True)
    close(kl, want, 1e-12)
    assert (kl >= 0).all()
    same = oracle.rl_eval(oracle.OP_KL_DIV, sh, dtype=oracle.F64, logits=a, ref_logits=a)
    assert (np.abs(same) < 1e-15).all()
    close(gq, ((np.exp(lq) - np.exp(lp)) / n).ravel(), 1e-12)
    per = (np.exp(lp) * (lp - lq)).sum(-1, keepdims=True)
    close(gp, (np.exp(lp) * (lp - lq - per) / n).ravel(), 1e-12)
    # finite differences on a few coordinates of the prediction, as fd_check does (1e-6 step)
    flat = a.ravel().copy()
    for i in (0, 7, 31, 59):
        hi, lo = flat.copy(), flat.copy()
        hi[i] += 1e-6
        lo[i] -= 1e-6
        f = lambda z: oracle.rl_eval(oracle.OP_KL_DIV, sh, dtype=oracle.F64, logits=z.reshape(sh), ref_logits=c).sum()
        assert abs((f(hi) - f(lo)) / 2e-6 - gq[i]) < 1e-7


def test_cross_entropy_options(oracle):
    # src/nn/tests/components.rs:551-588
    S, B, T, V = 2, 2, 3, 5
    n = B * T
    g = np.random.default_rng(72)
    a = g.uniform(-2, 2, (S, B, T, V))
    tg = g.integers(0, V, S * n)
    tg[1] = -100
    tg[7] = -100
    mask = (g.uniform(0, 1, S * n) < 0.8).astype(np.float64)
    sh = (S, B, T, V)
    a32 = a.astype(np.float32)
    bits = lambda x: np.asarray(x, np.float64).astype(np.float32).view(np.int32)
    # ignore_index = masked CE with those positions masked out (and any class as target), to the bit
    m2, tg2 = mask.copy(), tg.copy()
    m2[tg == -100] = 0.0
    tg2[tg == -100] = 0
    got = oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F32, logits=a32, tokens=tg, mask=mask, ignore_index=-100)
    want = oracle.rl_eval(oracle.OP_MASKED_CE, sh, dtype=oracle.F32, logits=a32, tokens=tg2, mask=m2)
    assert np.array_equal(bits(got), bits(want))
    # default options are the plain losses, to the bit
    assert np.array_equal(bits(oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F32, logits=a32, tokens=tg2, mask=mask)),
                          bits(oracle.rl_eval(oracle.OP_MASKED_CE, sh, dtype=oracle.F32, logits=a32, tokens=tg2, mask=mask)))
    assert np.array_equal(bits(oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F32, logits=a32, tokens=tg2)),
                          bits(oracle.rl_eval(oracle.OP_CE, sh, dtype=oracle.F32, logits=a32, tokens=tg2)))
    # label smoothing against the naive formula (f64)
    eps = 0.1
    got = oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F64, logits=a, tokens=tg, mask=mask, ignore_index=-100, smoothing=eps)
    lp = log_softmax(a).reshape(S * n, V)
    want = []
    for k in range(S):
        tot, cnt = 0.0, 0.0
        for i in range(n):
            j = k * n + i
            if tg[j] == -100 or mask[j] == 0.0:
                continue
            tot += (1 - eps) * -lp[j, tg[j]] + eps * -(lp[j].sum() / V)
            cnt += 1.0
        want.append(tot / max(cnt, 1.0))
    close(got, want, 1e-12)
    # its gradient: keep/count · (π − (1−ε)·onehot − ε/V)
    _, gd = oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F64, logits=a, tokens=tg, mask=mask, ignore_index=-100, smoothing=eps, upstream=np.ones(S))
    keep = (m2 != 0).astype(np.float64)
    count = np.maximum(keep.reshape(S, n).sum(1), 1.0).repeat(n)
    onehot = np.zeros((S * n, V))
    onehot[np.arange(S * n), tg2] = 1.0
    close(gd, ((keep / count)[:, None] * (np.exp(lp) - (1 - eps) * onehot - eps / V)).ravel(), 1e-12)
    import pytest

    with pytest.raises(RuntimeError, match="label smoothing"):
        oracle.rl_eval(oracle.OP_CE_WITH, sh, dtype=oracle.F64, logits=a, tokens=tg2, smoothing=1.5)
    with pytest.raises(RuntimeError, match="one_hot"):
        oracle.rl_eval(oracle.OP_CE, sh, dtype=oracle.F64, logits=a, tokens=tg)  # −100 without ignore_index


def test_forward_kl_is_the_expected_gradient_of_k3(oracle):
    # src/nn/tests/rl.rs:466-500: E_{x~π}[∇ k3] = ∇ KL(π_ref ‖ π) — the forward KL, `kl_div`
    V = 6
    g = np.random.default_rng(490)
    z, zr = g.uniform(-1.5, 1.5, V), g.uniform(-1.5, 1.5, V)
    sh = (1, 1, 1, V)
    _, fwd = oracle.rl_eval(oracle.OP_KL_DIV, sh, dtype=oracle.F64, logits=z, ref_logits=zr, upstream=np.ones(1))
    lp, lr = log_softmax(z), log_softmax(zr)
    expect = np.zeros(V)
    for x in range(V):
        _, gk = oracle.rl_eval(oracle.OP_KL_ESTIMATE, sh, dtype=oracle.F64, logits=z, tokens=[x], ref_logp=[lr[x]], estimator=oracle.K3, upstream=np.ones(1))
        expect += np.exp(lp[x]) * gk
    close(expect, fwd, 1e-10)
