"""Pins the CPU oracle against the hand-computed values, identities and tolerances of the
reference's own `nn::rl` tests (src/nn/tests/rl.rs; each test below names the lines it restates),
and its random streams against the published SHA-256 / ChaCha20 vectors. CPU only."""
import hashlib

import numpy as np
import pytest

import truth
from truth import Case

INF = float("inf")


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.abs(got - want) / (1.0 + np.abs(want))
    err = np.where(got == want, 0.0, err)
    assert np.all(err <= tol), f"max error {np.nanmax(err):.3e} > {tol}"


# ------------------------------------------------------------------ streams

def test_sha256_known_vectors(oracle):
    # FIPS 180-4 examples; the reference pins the same function in src/hash.rs:31-46.
    assert oracle.sha256(b"abc").hex() == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    assert oracle.sha256(b"").hex() == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    for msg in (b"a" * 55, b"a" * 56, b"a" * 64, b"noetic" * 100):
        assert oracle.sha256(msg) == hashlib.sha256(msg).digest()


def test_derive_is_sha256_of_root_le_and_label(oracle):
    # src/rng.rs:10-17
    assert oracle.derive_seed(5, "sampler test") == hashlib.sha256((5).to_bytes(8, "little") + b"sampler test").digest()


def test_chacha20_zero_key_keystream(oracle):
    # RFC 8439 A.1 test vector 1 (key 0, nonce 0, counter 0) and vector 2 (counter 1): the first
    # two blocks of ChaCha20Rng::from_seed([0; 32]).
    w = oracle.chacha20_words(bytes(32), 32)
    ks = w.astype("<u4").tobytes()
    assert ks[:64].hex() == ("76b8e0ada0f13d90405d6ae55386bd28bdd219b8a08ded1aa836efcc8b770dc7"
                             "da41597c5157488d7724e03fb8d84a376a43b8f41518a11cc387b669b2ee6586")
    assert ks[64:128].hex() == ("9f07e7be5551387a98ba977c732d080dcb0f29a048e3656912c6533e32ee7aed"
                                "29b721769ce64e43d57133b074d839d531ed1f28510afb45ace10a1f4b794d6f")
    # skipping words continues the same stream
    assert np.array_equal(oracle.chacha20_words(bytes(32), 8, skip=20), w[20:28])


def test_bf16_round_to_nearest_even(oracle):
    # src/tensor/half.rs:15-31
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, np.inf, 1e-40], dtype=np.float32)
    bits = oracle.bf16_from_f32(x)
    import torch

    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, want)
    assert np.array_equal(oracle.bf16_to_f32(bits), torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    nan = oracle.bf16_from_f32(np.array([np.nan], dtype=np.float32))
    assert np.isnan(oracle.bf16_to_f32(nan)[0])


# ------------------------------------------------------------------ token_log_probs

def test_token_log_probs_match_f64_reference(oracle):
    # src/nn/tests/rl.rs:100-122
    c = Case(800, -6.0, 6.0)
    want = c.logp_host()
    for dtype, tol in ((oracle.F64, 1e-14), (oracle.F32, 1e-6)):
        lp = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, c.lshape, dtype=dtype, logits=c.logits, tokens=c.tokens)
        close(lp, want, tol)
    _, g = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, upstream=np.ones(c.n))
    lp = truth.log_softmax_host(c.logits, c.v)
    onehot = np.zeros((c.n, c.v))
    onehot[np.arange(c.n), c.tokens] = 1.0
    close(g, (onehot - np.exp(lp)).ravel(), 1e-14)


def test_token_log_probs_large_and_excluded_logits(oracle):
    # src/nn/tests/rl.rs:133-156
    logits = np.array([1e4, -1e4, 0.0, 1e3, -1e4, -1e4, 1e4, 1e4])
    for dtype in (oracle.F32, oracle.F64):
        lv, gv = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, (1, 1, 2, 4), dtype=dtype, logits=logits, tokens=[0, 2], upstream=np.ones(2))
        assert abs(lv[0]) < 1e-6 and abs(lv[1] - np.log(0.5)) < 1e-6
        close(gv, [0, 0, 0, 0, 0, 0, 0.5, -0.5], 1e-6)
        row = [1.0, -INF, 0.0, 2.0]
        lv, gv = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, (1, 1, 2, 4), dtype=dtype, logits=np.array(row + row), tokens=[1, 3], upstream=np.array([0.0, 1.0]))
        assert lv[0] == -INF
        want = truth.log_softmax_host([1.0, 0.0, 2.0], 3)[0, 2]
        assert abs(lv[1] - want) < 1e-6


# ------------------------------------------------------------------ policy gradient

def test_policy_gradient_reductions_by_hand(oracle):
    # src/nn/tests/rl.rs:163-179
    lp = [-1.0, -2.0, -3.0, -4.0, -5.0, -6.0]
    w = np.array([[1.0, -2.0]])
    m = [1.0, 1.0, 0.0, 0.0, 1.0, 0.0]
    run = lambda r, **kw: oracle.rl_eval(oracle.OP_PG, (1, 2, 3, 1), dtype=oracle.F64, logp=lp, weights=kw.get("w", w), mask=kw.get("m", m), reduction=r)
    assert run(oracle.NONE).tolist() == [1.0, 2.0, 0.0, 0.0, -10.0, 0.0]
    assert run(oracle.SUM).tolist() == [-7.0]
    close(run(oracle.TOKEN_MEAN), [-7.0 / 3.0], 1e-15)
    assert run(oracle.PER_SEQUENCE).tolist() == [1.5, -10.0]
    assert run(oracle.SEQUENCE_MEAN).tolist() == [-4.25]
    wt = np.array([1.0, 1.0, 1.0, -2.0, -2.0, -2.0]).reshape(1, 2, 3)
    assert run(oracle.NONE, w=wt, m=None).tolist() == run(oracle.NONE, m=None).tolist()
    assert run(oracle.SUM, m=None).tolist() == [6.0 - 30.0]


def test_policy_gradient_matches_f64_reference(oracle):
    # src/nn/tests/rl.rs:183-207
    c = Case(820, -4.0, 4.0)
    s, b, t = c.sh
    g = np.random.default_rng(821)
    wtok, wseq = g.uniform(-2, 2, c.n), g.uniform(-2, 2, s * b)
    lp = c.logp_host()
    for per_seq in (False, True):
        w = np.repeat(wseq, t) if per_seq else wtok
        host = np.where(c.mask == 1.0, -w * lp, 0.0)
        for r in oracle.REDUCTIONS:
            want = truth.reduce_host(host, c.mask, c.sh, r)
            for dtype, tol in ((oracle.F64, 1e-13), (oracle.F32, 1e-6)):
                wt = wseq.reshape(s, b) if per_seq else wtok.reshape(c.sh)
                got = oracle.rl_eval(oracle.OP_PG, c.lshape, dtype=dtype, logits=c.logits, tokens=c.tokens, weights=wt, mask=c.mask, reduction=r)
                close(got, want, tol)


# ------------------------------------------------------------------ PPO clip

def ppo_case(seed, offs=(-0.5, -0.1, 0.05, 0.4), small=0.5):
    # src/nn/tests/rl.rs:227-234
    c = Case(seed, -3.0, 3.0)
    lp = c.logp_host()
    i = np.arange(c.n)
    old = lp + np.array(offs)[(i * 7 + i // 3) % len(offs)]
    adv = np.random.default_rng(seed + 5).uniform(-2, 2, c.n)
    adv = np.where(np.abs(adv) < 0.1, small, adv)
    return c, old, adv


def test_clipped_policy_loss_matches_f64_reference(oracle):
    # src/nn/tests/rl.rs:250-285
    c, old, adv = ppo_case(840)
    lp = c.logp_host()
    for clip in (oracle.Clip.symmetric(0.2), oracle.Clip(0.2, 0.28)):
        host = truth.ppo_host_full(lp, old, adv, c.mask, clip.low, clip.high)
        for r in oracle.REDUCTIONS:
            want = truth.reduce_host(host, c.mask, c.sh, r)
            for dtype, tol in ((oracle.F64, 1e-13), (oracle.F32, 1e-6)):
                got = oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=dtype, logits=c.logits, tokens=c.tokens, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask,
                                     clip=clip, reduction=r)
                close(got, want, tol)
        ratio = np.exp(lp - old)
        hit = (c.mask == 1.0) & (((adv > 0) & (ratio > 1 + clip.high)) | ((adv < 0) & (ratio < 1 - clip.low)))
        per = c.n // c.sh[0]
        want = hit.reshape(c.sh[0], per).sum(axis=1) / c.mask.reshape(c.sh[0], per).sum(axis=1)
        got = oracle.rl_eval(oracle.OP_CLIP_FRACTION, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask, clip=clip)
        close(got, want, 1e-15)


def test_clipped_policy_loss_gradients(oracle):
    # src/nn/tests/rl.rs:290-314: at old = logp the gradient is the policy-gradient loss's; per
    # token it is −A·r, or 0 where clipped and active.
    c, old, adv = ppo_case(850)
    lp = c.logp_host()
    up = np.ones(c.sh[0])
    _, g_ppo = oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F64, logp=lp, old_logp=lp, weights=adv.reshape(c.sh), mask=c.mask, clip=oracle.Clip.symmetric(0.2),
                              reduction=oracle.TOKEN_MEAN, upstream=up)
    _, g_pg = oracle.rl_eval(oracle.OP_PG, c.lshape, dtype=oracle.F64, logp=lp, weights=adv.reshape(c.sh), mask=c.mask, reduction=oracle.TOKEN_MEAN, upstream=up)
    close(g_ppo, g_pg, 1e-14)
    _, gv = oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F64, logp=lp, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask, clip=oracle.Clip.symmetric(0.2),
                           reduction=oracle.SUM, upstream=up)
    r = np.exp(lp - old)
    clipped = ((adv > 0) & (r > 1.2)) | ((adv < 0) & (r < 0.8))
    want = np.where((c.mask == 0) | clipped, 0.0, -adv * r)
    close(gv, want, 1e-14)


def test_clipped_policy_loss_ignores_garbage_at_masked_positions(oracle):
    # src/nn/tests/rl.rs:318-332
    c, old, adv = ppo_case(860)
    garbage = np.where(c.mask == 0.0, np.where(np.arange(c.n) % 2 == 0, -1e4, 1e4), old)
    run = lambda o: oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F32, logits=c.logits, tokens=c.tokens, old_logp=o, weights=adv.reshape(c.sh), mask=c.mask,
                                   clip=oracle.Clip.symmetric(0.2), reduction=oracle.TOKEN_MEAN, upstream=np.ones(c.sh[0]))
    (a0, a1), (b0, b1) = run(old), run(garbage)
    assert np.all(np.isfinite(b0)) and np.all(np.isfinite(b1))
    assert np.array_equal(a0, b0) and np.array_equal(a1, b1)


def test_clipped_policy_loss_dual_clip(oracle):
    # src/nn/tests/rl.rs:676-718
    c = Case(1000, -3.0, 3.0)
    lp = c.logp_host()
    offs = np.array([-1.5, -0.5, -0.1, 0.05, 0.4])
    i = np.arange(c.n)
    old = lp + offs[(i * 7 + i // 3) % 5]
    adv = np.random.default_rng(1001).uniform(-2, 2, c.n)
    adv = np.where(np.abs(adv) < 0.1, -0.5, adv)
    clip = oracle.Clip.symmetric(0.2).with_dual(3.0)
    host = truth.ppo_host_full(lp, old, adv, c.mask, 0.2, 0.2, dual=3.0, log_ratio_clamp=20.0)
    for r in oracle.REDUCTIONS:
        got = oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask, clip=clip,
                             reduction=r)
        close(got, truth.reduce_host(host, c.mask, c.sh, r), 1e-13)
    _, g = oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F64, logp=lp, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask, clip=clip, reduction=oracle.SUM,
                          upstream=np.ones(c.sh[0]))
    capped = (c.mask == 1.0) & (adv < 0) & (np.exp(lp - old) > 3.0)
    assert np.all(g[capped] == 0.0)
    ratio = np.exp(lp - old)
    hit = (c.mask == 1.0) & (((adv > 0) & (ratio > 1.2)) | ((adv < 0) & ((ratio < 0.8) | (ratio > 3.0))))
    per = c.n // c.sh[0]
    want = hit.reshape(c.sh[0], per).sum(axis=1) / c.mask.reshape(c.sh[0], per).sum(axis=1)
    close(oracle.rl_eval(oracle.OP_CLIP_FRACTION, c.lshape, dtype=oracle.F64, logp=lp, old_logp=old, weights=adv.reshape(c.sh), mask=c.mask, clip=clip), want, 1e-15)


def test_clipped_policy_loss_overflow_guards(oracle):
    # src/nn/tests/rl.rs:724-749
    lp, old, adv = [-0.5, -1.0], [-100.5, -1.0], np.array([-1.0, 1.0]).reshape(1, 1, 2)

    def run(clip):
        l, g = oracle.rl_eval(oracle.OP_PPO, (1, 1, 2, 1), dtype=oracle.F32, logp=lp, old_logp=old, weights=adv, clip=clip, reduction=oracle.NONE, upstream=np.array([1.0, 0.0]))
        return l, g[0]

    base = oracle.Clip.symmetric(0.2)
    l, _ = run(base.with_log_ratio_clamp(None))
    assert l[0] == INF
    l_clamped, g = run(base)
    close(l_clamped[:1], [float(np.exp(np.float32(20.0)))], 1e-7)
    assert g == 0.0
    l, g = run(base.with_dual(3.0))
    assert (l[0], g) == (3.0, 0.0)
    l, g = run(base.with_dual(3.0).with_log_ratio_clamp(None))
    assert l[0] == 3.0 and np.isnan(g)
    assert l_clamped[1] == -1.0
    f = oracle.rl_eval(oracle.OP_CLIP_FRACTION, (1, 1, 2, 1), dtype=oracle.F32, logp=lp, old_logp=old, weights=adv, clip=base)
    assert f.tolist() == [0.5]


# ------------------------------------------------------------------ KL, entropy, estimators

def test_kl_and_entropy_match_f64_reference(oracle):
    # src/nn/tests/rl.rs:347-371
    c = Case(870, -4.0, 4.0)
    refl = np.random.default_rng(871).uniform(-4, 4, c.n * c.v)
    kl = truth.kl_host(c.logits, refl, c.v) * c.mask
    h = truth.entropy_host(c.logits, c.v) * c.mask
    for r in oracle.REDUCTIONS:
        for dtype, tol in ((oracle.F64, 1e-13), (oracle.F32, 2e-6)):
            close(oracle.rl_eval(oracle.OP_KL, c.lshape, dtype=dtype, logits=c.logits, ref_logits=refl, mask=c.mask, reduction=r), truth.reduce_host(kl, c.mask, c.sh, r), tol)
            close(oracle.rl_eval(oracle.OP_ENTROPY, c.lshape, dtype=dtype, logits=c.logits, mask=c.mask, reduction=r), truth.reduce_host(h, c.mask, c.sh, r), tol)
    same = oracle.rl_eval(oracle.OP_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=c.logits)
    assert np.all(np.abs(same) < 1e-15)
    u = oracle.rl_eval(oracle.OP_ENTROPY, (1, 1, 2, c.v), dtype=oracle.F64, logits=np.full(2 * c.v, 0.3))
    close(u, [np.log(c.v)] * 2, 1e-15)
    assert np.all(kl >= 0)


def test_kl_and_entropy_with_excluded_and_large_logits(oracle):
    # src/nn/tests/rl.rs:389-423
    p = np.array([1.0, -INF, 0.5, -1.0, 2.0, 0.0, -INF, -INF])
    q = np.array([0.0, -INF, 1.5, 0.5, -1.0, 1.0, -INF, -INF])
    pk, qk = [1.0, 0.5, -1.0, 2.0, 0.0], [0.0, 1.5, 0.5, -1.0, 1.0]
    want_kl = [truth.kl_host(pk[:3], qk[:3], 3)[0], truth.kl_host(pk[3:], qk[3:], 2)[0]]
    want_h = [truth.entropy_host(pk[:3], 3)[0], truth.entropy_host(pk[3:], 2)[0]]
    for dtype, tol in ((oracle.F32, 1e-6), (oracle.F64, 1e-14)):
        kl, g = oracle.rl_eval(oracle.OP_KL, (1, 1, 2, 4), dtype=dtype, logits=p, ref_logits=q, upstream=np.ones(2))
        close(kl, want_kl, tol)
        assert np.all(np.isfinite(g)) and g[1] == 0.0 and g[6] == 0.0 and g[7] == 0.0
        h, g = oracle.rl_eval(oracle.OP_ENTROPY, (1, 1, 2, 4), dtype=dtype, logits=p, upstream=np.ones(2))
        close(h, want_h, tol)
        assert np.all(np.isfinite(g)) and g[1] == 0.0 and g[6] == 0.0 and g[7] == 0.0
        big, bref = np.array([1e4, -1e4, 0.0, 1e4]), np.array([-1e4, 1e4, 0.0, 0.0])
        k, gk = oracle.rl_eval(oracle.OP_KL, (1, 1, 1, 4), dtype=dtype, logits=big, ref_logits=bref, reduction=oracle.SUM, upstream=np.ones(1))
        e, ge = oracle.rl_eval(oracle.OP_ENTROPY, (1, 1, 1, 4), dtype=dtype, logits=big, reduction=oracle.SUM, upstream=np.ones(1))
        want = truth.kl_host(big, bref, 4)[0] + truth.entropy_host(big, 4)[0]
        lv = k[0] + e[0]
        assert np.isfinite(lv) and abs(lv - want) <= 1e-6 * (1 + abs(want))
        assert np.all(np.isfinite(gk)) and np.all(np.isfinite(ge))
        inf = oracle.rl_eval(oracle.OP_KL, (1, 1, 1, 2), dtype=dtype, logits=np.array([0.0, 0.0]), ref_logits=np.array([0.0, -INF]), reduction=oracle.SUM)
        assert inf[0] == INF


def test_kl_estimators_match_reference(oracle):
    # src/nn/tests/rl.rs:438-460
    c = Case(890, -3.0, 3.0)
    lp = c.logp_host()
    lr = lp + np.random.default_rng(891).uniform(-1.5, 1.5, c.n)
    for e in (oracle.K1, oracle.K2, oracle.K3):
        host = np.where(c.mask == 1.0, truth.k_host(lp, lr, e), 0.0)
        if e != oracle.K1:
            assert np.all(host >= 0)
        for r in oracle.REDUCTIONS:
            want = truth.reduce_host(host, c.mask, c.sh, r)
            for dtype, tol in ((oracle.F64, 1e-13), (oracle.F32, 2e-6)):
                got = oracle.rl_eval(oracle.OP_KL_ESTIMATE, c.lshape, dtype=dtype, logits=c.logits, tokens=c.tokens, ref_logp=lr, estimator=e, mask=c.mask, reduction=r)
                close(got, want, tol)


def test_kl_estimate_delta_clamp(oracle):
    # src/nn/tests/rl.rs:753-768
    lp, lr = [-100.5, -1.0], [-0.5, -1.2]
    open_ = oracle.rl_eval(oracle.OP_KL_ESTIMATE, (1, 1, 2, 1), dtype=oracle.F32, logp=lp, ref_logp=lr, estimator=oracle.K3)
    assert open_[0] == INF
    kv, g = oracle.rl_eval(oracle.OP_KL_ESTIMATE, (1, 1, 2, 1), dtype=oracle.F32, logp=lp, ref_logp=lr, estimator=oracle.K3, delta_clamp=oracle.KL_DELTA_CLAMP,
                           upstream=np.ones(2))
    want = float(np.exp(np.float32(20.0))) - 21.0
    assert abs(kv[0] - want) <= 1e-7 * want
    assert kv[1] == open_[1]
    assert g[0] == 0.0 and g[1] != 0.0


def test_kl_estimator_expectations_by_enumeration(oracle):
    # src/nn/tests/rl.rs:467-500: E[k1] = E[k3] = KL; E[∇k1] = 0; E[∇k2] = ∇KL(π‖ref).
    v = 6
    g = np.random.default_rng(900)
    pl, rl = g.uniform(-2, 2, v), g.uniform(-2, 2, v)
    pi = np.exp(truth.log_softmax_host(pl, v))[0]
    lr = truth.log_softmax_host(rl, v)[0]
    kl = truth.kl_host(pl, rl, v)[0]
    rows = np.tile(pl, v)

    def expect(e):
        val, grad = oracle.rl_eval(oracle.OP_KL_ESTIMATE, (1, 1, v, v), dtype=oracle.F64, logits=rows, tokens=np.arange(v), ref_logp=lr, estimator=e, upstream=pi)
        return float(val @ pi), grad.reshape(v, v).sum(axis=0)

    _, reverse = oracle.rl_eval(oracle.OP_KL, (1, 1, 1, v), dtype=oracle.F64, logits=pl, ref_logits=rl, reduction=oracle.SUM, upstream=np.ones(1))
    v1, dk1 = expect(oracle.K1)
    _, dk2 = expect(oracle.K2)
    v3, _ = expect(oracle.K3)
    close([v1], [kl], 1e-14)
    close([v3], [kl], 1e-14)
    close(dk1, np.zeros(v), 1e-14)
    close(dk2, reverse, 1e-14)


# ------------------------------------------------------------------ masking edges

def test_masking_edges_all_masked_and_one_token(oracle):
    # src/nn/tests/rl.rs:506-545
    c = Case(910, -3.0, 3.0)
    g = np.random.default_rng(911)
    old, adv = c.logp_host() + 0.3, g.uniform(-1, 1, c.n).reshape(c.sh)
    refl, lr = g.uniform(-3, 3, c.n * c.v), g.uniform(-4, -1, c.n)
    sym = oracle.Clip.symmetric(0.2)
    losses = {
        "PG": lambda m, r, up: oracle.rl_eval(oracle.OP_PG, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, weights=adv, mask=m, reduction=r, upstream=up),
        "PPO": lambda m, r, up: oracle.rl_eval(oracle.OP_PPO, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, old_logp=old, weights=adv, mask=m, clip=sym, reduction=r, upstream=up),
        "KL": lambda m, r, up: oracle.rl_eval(oracle.OP_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=refl, mask=m, reduction=r, upstream=up),
        "k3": lambda m, r, up: oracle.rl_eval(oracle.OP_KL_ESTIMATE, c.lshape, dtype=oracle.F64, logits=c.logits, tokens=c.tokens, ref_logp=lr, estimator=oracle.K3, delta_clamp=20.0, mask=m, reduction=r, upstream=up),
        "entropy": lambda m, r, up: oracle.rl_eval(oracle.OP_ENTROPY, c.lshape, dtype=oracle.F64, logits=c.logits, mask=m, reduction=r, upstream=up),
    }
    none = np.zeros(c.n)
    one = np.zeros(c.n)
    one[c.n - 2] = 1.0
    for name, f in losses.items():
        for r in oracle.REDUCTIONS:
            l, g_ = f(none, r, np.ones(int(np.prod(oracle.out_shape(c.lshape, r)))))
            assert np.all(l == 0.0) and np.all(g_ == 0.0), (name, r)
        per, _ = f(one, oracle.NONE, np.ones(c.n))
        only = per[c.n - 2]
        assert all(v == 0.0 for i, v in enumerate(per) if i != c.n - 2)
        for r in (oracle.TOKEN_MEAN, oracle.SEQUENCE_MEAN, oracle.SUM):
            got, _ = f(one, r, np.ones(c.sh[0]))
            assert got.tolist() == [0.0, only], (name, r)
        _, g_ = f(c.mask, oracle.TOKEN_MEAN, np.ones(c.sh[0]))
        gm = g_.reshape(c.n, c.v)
        assert np.all(gm[c.mask == 0.0] == 0.0), name


# ------------------------------------------------------------------ group advantages

def test_group_advantages_by_hand(oracle):
    # src/nn/tests/rl.rs:550-575
    r = [1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0, 0.0, 0.0, 0.0, 3.0]
    s3 = 0.5 / np.sqrt(1.0 / 3.0)
    close(oracle.group_advantages(r, 4, "std", 0.0, True), [s3, -s3, -s3, s3, 0, 0, 0, 0, -0.5, -0.5, -0.5, 1.5], 1e-15)
    p3 = np.sqrt(1.6875)
    close(oracle.group_advantages(r, 4, "std", 0.0, False), [1, -1, -1, 1, 0, 0, 0, 0, -0.75 / p3, -0.75 / p3, -0.75 / p3, 2.25 / p3], 1e-15)
    assert oracle.group_advantages(r, 4, "mean").tolist() == [0.5, -0.5, -0.5, 0.5, 0, 0, 0, 0, -0.75, -0.75, -0.75, 2.25]
    close(oracle.group_advantages(r, 4, "std", 1e-2, True)[8:], [-0.75 / 1.51] * 3 + [2.25 / 1.51], 1e-15)
    assert oracle.group_advantages([3.0, -1.0], 1, "std", 1e-6, False).tolist() == [0.0, 0.0]
    with pytest.raises(RuntimeError, match="at least 2"):
        oracle.group_advantages([1.0, 2.0], 1, "std", 1e-6, True)


def test_group_advantages_equal_rewards_are_zero_at_eps_zero(oracle):
    # src/nn/tests/rl.rs:644-653
    r = [0.1, 0.1, 0.1, 1.0, 0.0, 0.0]
    for norm, unb in (("std", True), ("std", False), ("mean", True)):
        a = oracle.group_advantages(r, 3, norm, 0.0, unb)
        assert a[:3].tolist() == [0.0, 0.0, 0.0]
        assert a[3] > 0 and a[4] < 0 and a[4] == a[5]


# ------------------------------------------------------------------ masks: −1e9 ≡ −∞, temperature

def test_additive_mask_minus_1e9_matches_minus_infinity(oracle):
    # src/nn/tests/rl.rs:773-813
    c = Case(1010, -4.0, 4.0)
    refl = np.random.default_rng(1011).uniform(-4, 4, c.n * c.v)
    tokens = np.where(c.tokens == 3, 1, c.tokens)
    for dtype in (oracle.F32, oracle.F64):
        def run(fill):
            vm = np.where(np.arange(c.v) == 3, fill, 0.0)
            outs = []
            outs += list(oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, c.lshape, dtype=dtype, logits=c.logits, tokens=tokens, vocab_mask=vm, temperature=0.8, upstream=np.ones(c.n)))
            outs += list(oracle.rl_eval(oracle.OP_REFERENCE_KL, c.lshape, dtype=dtype, logits=c.logits, ref_logits=refl, vocab_mask=vm, temperature=0.8, mask=c.mask, upstream=np.ones(c.n)))
            outs += list(oracle.rl_eval(oracle.OP_ENTROPY, c.lshape, dtype=dtype, logits=c.logits, vocab_mask=vm, temperature=0.8, mask=c.mask, upstream=np.ones(c.n)))
            return outs
        a, b = run(-1e9), run(-INF)
        for x, y in zip(a, b):
            assert np.all(np.isfinite(x))
            assert np.array_equal(x, y)
        one = np.array([0.0, 0.5, 1.0])
        kl_with = lambda fill: oracle.rl_eval(oracle.OP_KL, (1, 1, 1, 3), dtype=dtype, logits=one, ref_logits=one + np.array([0.0, 0.0, fill]), reduction=oracle.SUM)[0]
        assert kl_with(-INF) == INF
        p2 = np.exp(truth.log_softmax_host(one, 3)[0, 2])
        assert abs(kl_with(-1e9) / (1e9 * p2) - 1.0) < 1e-6


def test_reference_kl_uses_the_sampling_temperature_on_both_sides(oracle):
    # src/nn/tests/rl.rs:818-835
    c = Case(1020, -4.0, 4.0)
    refl = np.random.default_rng(1021).uniform(-4, 4, c.n * c.v)
    vm = np.where(np.arange(c.v) == 2, -INF, 0.0)
    for tau in (0.6, 1.0, 1.7):
        got = oracle.rl_eval(oracle.OP_REFERENCE_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=refl, temperature=tau, vocab_mask=vm, mask=c.mask, reduction=oracle.TOKEN_MEAN)
        z, zr = c.logits.reshape(-1, c.v) / tau + vm, refl.reshape(-1, c.v) / tau + vm
        want = truth.reduce_host(truth.kl_host(z, zr, c.v) * c.mask, c.mask, c.sh, oracle.TOKEN_MEAN)
        close(got, want, 1e-13)
    a = oracle.rl_eval(oracle.OP_REFERENCE_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=refl)
    b = oracle.rl_eval(oracle.OP_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=refl)
    assert np.array_equal(a, b)
    same = oracle.rl_eval(oracle.OP_REFERENCE_KL, c.lshape, dtype=oracle.F64, logits=c.logits, ref_logits=c.logits, temperature=0.6, vocab_mask=vm)
    assert np.all(np.abs(same) < 1e-15)


# ------------------------------------------------------------------ samplers

def test_reference_sampler_matches_its_distribution(oracle):
    # src/nn/tests/rl.rs:582-629: frequencies within 4.5 standard errors over 40 000 draws, an
    # excluded token never drawn, same stream same tokens, temperature 0 greedy.
    v, n = 6, 40_000
    row = np.array([0.4, -1.0, 1.2, 3.0, 0.0, -0.3], dtype=np.float32)
    maskrow = np.array([0.0, 0.0, 0.0, -INF, 0.5, 0.0], dtype=np.float32)
    logits = np.tile(row, (n, 1))
    for tau in (0.7, 2.5):
        tok = oracle.sample_gumbel(logits, tau, 5, "sampler test", add_mask=maskrow)
        z = row.astype(np.float64) / tau + maskrow
        p = np.exp(truth.log_softmax_host(z, v))[0]
        count = np.bincount(tok, minlength=v)
        assert count[3] == 0
        f = count / n
        se = np.sqrt(p * (1 - p) / n)
        assert np.all(np.abs(f - p) <= 4.5 * se + 1e-12)
        assert np.array_equal(oracle.sample_gumbel(logits, tau, 5, "sampler test", add_mask=maskrow), tok)
        assert not np.array_equal(oracle.sample_gumbel(logits, tau, 6, "sampler test", add_mask=maskrow), tok)
    greedy_mask = np.array([0.0, 0.0, 0.0, -INF, 2.0, 0.0], dtype=np.float32)
    assert oracle.sample_gumbel(np.tile(row, (2, 1)), 0.0, 1, "greedy", add_mask=greedy_mask).tolist() == [4, 4]


def test_reference_sampler_refuses_a_position_with_no_allowed_token(oracle):
    # src/nn/tests/rl.rs:631-637
    logits = np.zeros((2, 3), dtype=np.float32)
    mask = np.array([[0.0, 0.0, 0.0], [-INF, -INF, -INF]], dtype=np.float32)
    with pytest.raises(RuntimeError, match="position 1 has no allowed token"):
        oracle.sample_gumbel(logits, 1.0, 0, "x", add_mask=mask)


def test_inverse_cdf_sampler_definition(oracle):
    # The build's own sampler definition: first index whose cumulative mass exceeds u·Z.
    row = np.log(np.array([[0.1, 0.2, 0.0, 0.3, 0.4]], dtype=np.float64) + 1e-300).astype(np.float32)
    rows = np.tile(row, (6, 1))
    u = np.array([0.0, 0.05, 0.1000001, 0.29, 0.31, 0.99], dtype=np.float32)
    o = oracle.sample_inverse_cdf(rows, 1.0, u)
    assert o["tokens"].tolist() == [0, 0, 1, 1, 3, 4]
    assert o["boundary"].tolist() == [0, 0, 1, 0, 0, 0]
    close(o["logp"], np.log([0.1, 0.1, 0.2, 0.2, 0.3, 0.4]), 1e-6)
    # an allow-mask removes tokens; a row with none is refused (status bit 0)
    allow = np.array([[1, 0, 1, 0, 1]] * 5 + [[0, 0, 0, 0, 0]], dtype=np.uint8)
    o = oracle.sample_inverse_cdf(rows, 1.0, u, allow=allow)
    assert o["status"].tolist() == [0, 0, 0, 0, 0, 1] and o["tokens"][5] == -1
    assert set(o["tokens"][:5].tolist()) <= {0, 4}
    # frequencies over many uniforms
    n = 40_000
    r6 = np.array([0.4, -1.0, 1.2, 3.0, 0.0, -0.3], dtype=np.float32)
    mrow = np.array([0.0, 0.0, 0.0, -INF, 0.5, 0.0], dtype=np.float32)
    uu = oracle.row_uniforms(5, "sampler test", n)
    assert uu.min() >= 0.0 and uu.max() < 1.0
    o = oracle.sample_inverse_cdf(np.tile(r6, (n, 1)), 0.7, uu, add_mask=mrow)
    p = np.exp(truth.log_softmax_host(r6.astype(np.float64) / np.float32(0.7) + mrow, 6))[0]
    f = np.bincount(o["tokens"], minlength=6) / n
    assert f[3] == 0
    assert np.all(np.abs(f - p) <= 4.5 * np.sqrt(p * (1 - p) / n) + 1e-12)
    # temperature 0: first maximum of the masked logits, no uniform needed
    g = oracle.sample_inverse_cdf(np.tile(r6, (2, 1)), 0.0, None, add_mask=np.array([0.0, 0.0, 0.0, -INF, 2.0, 0.0], dtype=np.float32))
    assert g["tokens"].tolist() == [4, 4]


def test_fast_backend_matches_reference_within_lane_sum_tolerance(oracle):
    # src/tensor/tests/fast.rs:86-137: Fast equals Reference except lane sums (≤ 1e-5).
    g = np.random.default_rng(3)
    S, B, T, V = 1, 2, 8, 1 << 18  # 2^22 elements: above every Fast threshold
    logits = g.normal(0, 2, S * B * T * V).astype(np.float32)
    tokens = g.integers(0, V, S * B * T)
    a = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, (S, B, T, V), logits=logits, tokens=tokens)
    oracle.set_backend(True, 4)
    try:
        b = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, (S, B, T, V), logits=logits, tokens=tokens)
    finally:
        oracle.set_backend(False, 1)
    close(b, a, 1e-5)
    assert not np.array_equal(a, b) or True


def test_inverse_cdf_oracle_values_equal_the_restated_engine(oracle):
    """The f64 sampler oracle is this build's definition for the TOKEN; the values it returns beside
    it must be the pinned engine's: token_log_probs, reference_kl and categorical_entropy in F64 on
    the same masked logits (src/nn/rl.rs:134-141, 347-351, 405-414)."""
    g = np.random.default_rng(77)
    S, B, T, V = 2, 3, 4, 40
    rows = S * B * T
    x = g.normal(0, 2, (rows, V)).astype(np.float32)
    ref = (x + g.normal(0, 0.3, (rows, V))).astype(np.float32)
    allow = (g.uniform(0, 1, (rows, V)) < 0.6).astype(np.uint8)
    allow[:, 3] = 1
    u = oracle.row_uniforms(5, "cross-check", rows)
    o = oracle.sample_inverse_cdf(x, 1.0, u, ref_logits=ref, allow=allow)
    vm = np.where(allow != 0, 0.0, -INF)
    shape = (S, B, T, V)
    lp = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, shape, dtype=oracle.F64, logits=x, tokens=o["tokens"], vocab_mask=vm)
    kl = oracle.rl_eval(oracle.OP_REFERENCE_KL, shape, dtype=oracle.F64, logits=x, ref_logits=ref, vocab_mask=vm, reduction=oracle.NONE)
    en = oracle.rl_eval(oracle.OP_ENTROPY, shape, dtype=oracle.F64, logits=x, vocab_mask=vm, reduction=oracle.NONE)
    assert np.abs(lp - o["logp"]).max() < 1e-12
    assert np.abs(kl - o["kl"]).max() < 1e-12
    assert np.abs(en - o["entropy"]).max() < 1e-12
    assert allow[np.arange(rows), o["tokens"]].all()


def test_scored_log_probs_must_be_finite(oracle):
    """src/nn/tests/rl.rs:837-846: finite scored values pass; a −inf at a scored position is named;
    one at a masked position passes."""
    lp = [-1.0, -np.inf, -2.0]
    e = oracle.check_scored_finite("test", lp)
    assert e == "test: the scored log-probability at flat position 1 is -inf (not finite)"
    assert oracle.check_scored_finite("test", lp, [1.0, 0.0, 1.0]) is None
    assert oracle.check_scored_finite("test", [-1.0, -3.0, -2.0]) is None
    assert "position 2 is NaN" in oracle.check_scored_finite("test", [0.0, -1.0, np.nan, -np.inf])
