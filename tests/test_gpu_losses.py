"""GPU parity of the `nn::rl` losses against the CPU restatement of `Cpu(Reference)`, restating the
reference's own device test (src/nn/tests/gpu/rl.rs:25-138): S 2 · B 8 · T 12 · V 24 with ±1e4 and
−∞ logits and masked positions, eleven losses, values within 1e-5 and gradients within 1e-4 of
CpuRef by |Δ|/(1+|ref|), masked positions with exactly zero gradient, bitwise run to run. Plus
the hand-computed token-level cases of src/nn/tests/rl.rs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

INF = float("inf")
SH = (2, 8, 12)
V = 24


def dev():
    return torch.device("cuda:0")


def t32(a, shape=None):
    t = torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dev())
    return t.reshape(shape).contiguous() if shape is not None else t


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64).ravel(), np.asarray(b, dtype=np.float64).ravel()
    assert a.shape == b.shape
    e = np.abs(a - b) / (1.0 + np.abs(b))
    e = np.where(a == b, 0.0, e)
    return float(np.max(e)) if e.size else 0.0


def data():
    g = np.random.default_rng(950)
    n = int(np.prod(SH))
    logits = g.uniform(-6, 6, (n, V))
    refl = g.uniform(-6, 6, (n, V))
    tokens = g.integers(0, V, n)
    for i in range(0, n, 5):
        t = tokens[i]
        a, b = (t + 1) % V, (t + 2) % V
        logits[i, a] = -INF
        refl[i, a] = -INF
        logits[i, b] = 1e4 if i % 2 == 0 else -1e4
    mask = (g.uniform(0, 1, n) < 0.75).astype(np.float64)
    T = SH[2]
    mask[3 * T:4 * T] = 0.0
    old = g.uniform(-8, -0.5, n)
    adv = g.uniform(-2, 2, n)
    mx = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - mx).sum(axis=1, keepdims=True)) + mx
    lr = (logits - lse)[np.arange(n), tokens] + g.uniform(-1.5, 1.5, n)
    return dict(logits=logits.astype(np.float32), refl=refl.astype(np.float32), tokens=tokens, mask=mask, old=old, adv=adv, lr=lr)


def cases(d, orc, rl):
    """(name, oracle kwargs, device closure) for the eleven losses of the reference's device test."""
    S, B, T = SH
    lsh = (S, B, T, V)
    vmask = np.where(np.arange(V) % 5 == 4, -1e9, 0.0)
    x = t32(d["logits"], lsh)
    refl = t32(d["refl"], lsh)
    tok = torch.from_numpy(d["tokens"]).to(dev()).reshape(SH)
    m, old, adv, lr = t32(d["mask"], SH), t32(d["old"], SH), t32(d["adv"], SH), t32(d["lr"], SH)
    advs_np = d["adv"][: S * B].reshape(S, B)
    advs = t32(advs_np)
    vm = t32(vmask, (1, V))
    base = dict(logits=d["logits"], tokens=d["tokens"], mask=d["mask"])
    O, R = orc, rl
    return [
        ("token_log_probs", dict(op=O.OP_TOKEN_LOG_PROBS, **base), lambda: R.token_log_probs(x, tok, mask=m)),
        ("pg token-mean", dict(op=O.OP_PG, weights=d["adv"].reshape(SH), reduction=O.TOKEN_MEAN, **base), lambda: R.policy_gradient_loss(x, tok, adv, m, R.TOKEN_MEAN)),
        ("pg per-sequence weights, none", dict(op=O.OP_PG, weights=advs_np, reduction=O.NONE, **base), lambda: R.policy_gradient_loss(x, tok, advs, m, R.NONE)),
        ("ppo sum", dict(op=O.OP_PPO, old_logp=d["old"], weights=d["adv"].reshape(SH), clip=O.Clip(0.2, 0.28), reduction=O.SUM, **base),
         lambda: R.clipped_policy_loss(x, tok, old, adv, m, R.Clip(0.2, 0.28), R.SUM)),
        ("kl sequence-mean", dict(op=O.OP_KL, logits=d["logits"], ref_logits=d["refl"], mask=d["mask"], reduction=O.SEQUENCE_MEAN),
         lambda: R.categorical_kl(x, refl, m, R.SEQUENCE_MEAN)),
        ("k1 per-sequence", dict(op=O.OP_KL_ESTIMATE, ref_logp=d["lr"], estimator=O.K1, reduction=O.PER_SEQUENCE, **base), lambda: R.kl_estimate(x, tok, lr, R.K1, None, m, R.PER_SEQUENCE)),
        ("k2 per-sequence", dict(op=O.OP_KL_ESTIMATE, ref_logp=d["lr"], estimator=O.K2, reduction=O.PER_SEQUENCE, **base), lambda: R.kl_estimate(x, tok, lr, R.K2, None, m, R.PER_SEQUENCE)),
        ("k3 per-sequence", dict(op=O.OP_KL_ESTIMATE, ref_logp=d["lr"], estimator=O.K3, delta_clamp=20.0, reduction=O.PER_SEQUENCE, **base),
         lambda: R.kl_estimate(x, tok, lr, R.K3, 20.0, m, R.PER_SEQUENCE)),
        ("ppo dual clip, no log-ratio clamp, token-mean",
         dict(op=O.OP_PPO, old_logp=d["old"], weights=d["adv"].reshape(SH), clip=O.Clip.symmetric(0.2).with_dual(3.0).with_log_ratio_clamp(None), reduction=O.TOKEN_MEAN, **base),
         lambda: R.clipped_policy_loss(x, tok, old, adv, m, R.Clip.symmetric(0.2).with_dual(3.0).with_log_ratio_clamp(None), R.TOKEN_MEAN)),
        ("reference kl τ 0.7 with a −1e9 vocabulary mask, token-mean",
         dict(op=O.OP_REFERENCE_KL, logits=d["logits"], ref_logits=d["refl"], mask=d["mask"], temperature=0.7, vocab_mask=vmask, reduction=O.TOKEN_MEAN),
         lambda: R.reference_kl(x, refl, 0.7, vm, m, R.TOKEN_MEAN)),
        ("entropy token-mean", dict(op=O.OP_ENTROPY, logits=d["logits"], mask=d["mask"], reduction=O.TOKEN_MEAN), lambda: R.categorical_entropy(x, m, R.TOKEN_MEAN)),
    ]


def test_rl_losses_on_the_device(oracle):
    from noetic_tensor_b200 import rl

    d = data()
    lsh = (*SH, V)
    worst = [0.0, 0.0]
    for name, okw, run in cases(d, oracle, rl):
        okw = dict(okw)
        op = okw.pop("op")
        red = okw.get("reduction", oracle.NONE)
        n_out = int(np.prod(oracle.out_shape(lsh, red)))
        up = np.random.default_rng(9).uniform(-1, 1, n_out)
        want_v, want_g = oracle.rl_eval(op, lsh, dtype=oracle.F32, upstream=up, **okw)
        loss = run()
        got_v = loss.value.cpu().numpy()
        got_g = loss.backward(torch.from_numpy(up.astype(np.float32)).to(dev()).reshape(loss.value.shape)).cpu().numpy()
        assert np.isfinite(got_v).all() and np.isfinite(got_g).all(), name
        ev, eg = rel(got_v, want_v), rel(got_g, want_g)
        assert ev <= 1e-5, f"{name} value: {ev:e} from CpuRef"
        assert eg <= 1e-4, f"{name} gradient: {eg:e} from CpuRef"
        worst = [max(worst[0], ev), max(worst[1], eg)]
        gm = got_g.reshape(-1, V)
        assert (gm[d["mask"] == 0.0] == 0.0).all(), f"{name}: a masked position has a gradient"
        again = run()
        assert torch.equal(again.value.view(torch.int32), loss.value.view(torch.int32)), f"{name} value run to run"
        g2 = again.backward(torch.from_numpy(up.astype(np.float32)).to(dev()).reshape(loss.value.shape))
        assert np.array_equal(g2.cpu().numpy().view(np.int32), got_g.view(np.int32)), f"{name} gradient run to run"
    print(f"rl losses: values within {worst[0]:.1e} and gradients within {worst[1]:.1e} of CpuRef")


def tok_case(S, B, T):
    return (S, B, T)


def test_policy_gradient_reductions_by_hand():
    # src/nn/tests/rl.rs:163-179
    from noetic_tensor_b200 import capi, ops

    lp = t32([-1, -2, -3, -4, -5, -6], (1, 2, 3))
    w = t32([[1.0, -2.0]])
    m = t32([1, 1, 0, 0, 1, 0], (1, 2, 3))
    per, dl = ops.token_loss(capi.LOSS_PG, lp, weights=w, mask=m)
    assert per.cpu().ravel().tolist() == [1.0, 2.0, 0.0, 0.0, -10.0, 0.0]
    assert dl.cpu().ravel().tolist() == [-1.0, -1.0, 0.0, 0.0, 2.0, 0.0]
    red = lambda r: ops.reduce_tokens(per, m, r).cpu().ravel().tolist()
    assert red(capi.REDUCE_SUM) == [-7.0]
    assert abs(red(capi.REDUCE_TOKEN_MEAN)[0] - (-7.0 / 3.0)) < 1e-6
    assert red(capi.REDUCE_PER_SEQUENCE) == [1.5, -10.0]
    assert red(capi.REDUCE_SEQUENCE_MEAN) == [-4.25]
    per2, _ = ops.token_loss(capi.LOSS_PG, lp, weights=w)
    assert ops.reduce_tokens(per2, None, capi.REDUCE_SUM).cpu().tolist() == [6.0 - 30.0]
    # a log-prob tensor that feeds two losses: the second derivative is added into the first
    ref = t32([-1.5, -2, -2, -4, -4, -7], (1, 2, 3))
    _, dk = ops.token_loss(capi.LOSS_K1, lp, other=ref, mask=m)
    _, both = ops.token_loss(capi.LOSS_K1, lp, other=ref, mask=m, accumulate_into=dl.clone())
    assert torch.equal(both, dl + dk) and both.cpu().ravel().tolist() == [0.0, 0.0, 0.0, 0.0, 3.0, 0.0]


def test_clipped_policy_loss_overflow_guards():
    # src/nn/tests/rl.rs:724-749
    from noetic_tensor_b200 import capi, ops

    lp, old, adv = t32([-0.5, -1.0], (1, 1, 2)), t32([-100.5, -1.0], (1, 1, 2)), t32([-1.0, 1.0], (1, 1, 2))

    def run(dual=None, clamp=20.0):
        l, g = ops.token_loss(capi.LOSS_PPO, lp, other=old, weights=adv, clip_low=0.2, clip_high=0.2, dual=dual, clamp=clamp)
        return l.cpu().numpy(), g.cpu().numpy().ravel()[0]

    l, _ = run(clamp=None)
    assert l.ravel()[0] == INF
    l, g = run()
    assert abs(l.ravel()[0] - float(np.exp(np.float32(20.0)))) <= 1e-7 * float(np.exp(np.float32(20.0))) * 4 and g == 0.0
    assert l.ravel()[1] == -1.0
    l, g = run(dual=3.0)
    assert (l.ravel()[0], g) == (3.0, 0.0)
    l, g = run(dual=3.0, clamp=None)
    assert l.ravel()[0] == 3.0 and np.isnan(g)
    f = ops.clip_fraction(lp, old, adv, clip_low=0.2, clip_high=0.2, clamp=20.0)
    assert f.cpu().tolist() == [0.5]


def test_kl_estimate_delta_clamp():
    # src/nn/tests/rl.rs:753-768
    from noetic_tensor_b200 import capi, ops

    lp, lr = t32([-100.5, -1.0], (1, 1, 2)), t32([-0.5, -1.2], (1, 1, 2))
    open_, _ = ops.token_loss(capi.LOSS_K3, lp, other=lr)
    assert open_.cpu().ravel()[0].item() == INF
    kv, g = ops.token_loss(capi.LOSS_K3, lp, other=lr, clamp=20.0)
    want = float(np.exp(np.float32(20.0))) - 21.0
    assert abs(kv.cpu().ravel()[0].item() - want) <= 1e-6 * want
    assert kv.cpu().ravel()[1].item() == open_.cpu().ravel()[1].item()
    assert g.cpu().ravel()[0].item() == 0.0 and g.cpu().ravel()[1].item() != 0.0


@pytest.mark.parametrize("shape", [(2, 3, 4), (3, 5, 300), (1, 1, 1), (4, 64, 1024)])
def test_token_losses_and_reductions_match_cpu_reference(oracle, shape):
    """Every loss kind × reduction on random [S,B,T] values (a fully masked sequence, a one-token
    sequence, per-sequence and per-token weights) against the f32 CpuRef restatement."""
    from noetic_tensor_b200 import capi, ops

    S, B, T = shape
    n = S * B * T
    g = np.random.default_rng(n)
    lp = g.uniform(-8, -0.1, n)
    old = lp + g.choice([-1.5, -0.5, -0.1, 0.05, 0.4], n)
    lr = lp + g.uniform(-1.5, 1.5, n)
    adv = g.uniform(-2, 2, n)
    advs = g.uniform(-2, 2, S * B)
    mask = (g.uniform(0, 1, n) < 0.7).astype(np.float64)
    mask[:T] = 0.0
    if T > 1:
        mask[-T:] = 0.0
        mask[-2] = 1.0
    lsh = (S, B, T, 1)
    kinds = [
        ("pg", capi.LOSS_PG, dict(weights=adv.reshape(shape)), dict(op=oracle.OP_PG, weights=adv.reshape(shape))),
        ("pg-seq", capi.LOSS_PG, dict(weights=advs.reshape(S, B)), dict(op=oracle.OP_PG, weights=advs.reshape(S, B))),
        ("ppo", capi.LOSS_PPO, dict(other=old, weights=adv.reshape(shape), clip_low=0.2, clip_high=0.28, clamp=20.0),
         dict(op=oracle.OP_PPO, old_logp=old, weights=adv.reshape(shape), clip=oracle.Clip(0.2, 0.28))),
        ("ppo-dual", capi.LOSS_PPO, dict(other=old, weights=advs.reshape(S, B), clip_low=0.2, clip_high=0.2, dual=3.0, clamp=20.0),
         dict(op=oracle.OP_PPO, old_logp=old, weights=advs.reshape(S, B), clip=oracle.Clip.symmetric(0.2).with_dual(3.0))),
        ("k1", capi.LOSS_K1, dict(other=lr), dict(op=oracle.OP_KL_ESTIMATE, ref_logp=lr, estimator=oracle.K1)),
        ("k2", capi.LOSS_K2, dict(other=lr, clamp=1.0), dict(op=oracle.OP_KL_ESTIMATE, ref_logp=lr, estimator=oracle.K2, delta_clamp=1.0)),
        ("k3", capi.LOSS_K3, dict(other=lr, clamp=20.0), dict(op=oracle.OP_KL_ESTIMATE, ref_logp=lr, estimator=oracle.K3, delta_clamp=20.0)),
    ]
    lpt, mt = t32(lp, shape), t32(mask, shape)
    for name, kind, kw, okw in kinds:
        kw = {k: (t32(v, v.shape if hasattr(v, "shape") and v.ndim > 1 else shape) if isinstance(v, np.ndarray) else v) for k, v in kw.items()}
        okw = dict(okw)
        op = okw.pop("op")
        for use_mask in (True, False):
            m_t, m_np = (mt, mask) if use_mask else (None, None)
            per, _ = ops.token_loss(kind, lpt, mask=m_t, want_grad=False, **kw)
            for r in range(5):
                n_out = int(np.prod(oracle.out_shape(lsh, r)))
                up = g.uniform(-1, 1, n_out)
                want_v, want_g = oracle.rl_eval(op, lsh, dtype=oracle.F32, logp=lp, mask=m_np, reduction=r, upstream=up, **okw)
                val = ops.reduce_tokens(per, m_t, r)
                d_per = ops.reduce_tokens_backward(shape, m_t, r, t32(up, val.shape))
                _, gl = ops.token_loss(kind, lpt, mask=m_t, upstream=d_per, **kw)
                # a long signed sum cancels: the f32 reference itself is then only accurate to
                # eps·Σ|terms|, so the reduced value is held to the f64 path with that allowance,
                # and to CpuRef where the sums are short
                true_v = oracle.rl_eval(op, lsh, dtype=oracle.F64, logp=lp, mask=m_np, reduction=r, **okw)
                slack = 0.0 if r == 0 else 2e-7 * float(per.abs().sum().item()) / S
                dv = np.abs(val.cpu().numpy().astype(np.float64).ravel() - true_v)
                assert (dv <= 1e-5 * (1.0 + np.abs(true_v)) + slack).all(), (name, r, use_mask, float(dv.max()))
                if n <= 64:
                    assert rel(val.cpu().numpy(), want_v) <= 1e-5, (name, r, use_mask)
                assert rel(gl.cpu().numpy(), want_g) <= 1e-5, (name, r, use_mask)
                if use_mask:
                    assert (gl.cpu().numpy().ravel()[mask == 0.0] == 0.0).all()
        if kind == capi.LOSS_PPO:
            cf = ops.clip_fraction(lpt, kw["other"], kw["weights"], mask=mt, clip_low=kw["clip_low"], clip_high=kw["clip_high"], dual=kw.get("dual"), clamp=kw.get("clamp"))
            want = oracle.rl_eval(oracle.OP_CLIP_FRACTION, lsh, dtype=oracle.F32, logp=lp, mask=mask, **okw)
            assert rel(cf.cpu().numpy(), want) <= 1e-6, name


def test_all_masked_and_one_token(oracle):
    # src/nn/tests/rl.rs:506-545: every position masked → value and gradient exactly 0
    from noetic_tensor_b200 import rl

    g = np.random.default_rng(910)
    S, B, T, Vv = 2, 3, 4, 5
    x = t32(g.uniform(-3, 3, (S, B, T, Vv)))
    refl = t32(g.uniform(-3, 3, (S, B, T, Vv)))
    tok = torch.from_numpy(g.integers(0, Vv, (S, B, T))).to(dev())
    adv = t32(g.uniform(-1, 1, (S, B, T)))
    none = torch.zeros(S, B, T, device=dev())
    one = none.clone()
    one.view(-1)[-2] = 1.0
    fns = {
        "PG": lambda m, r: rl.policy_gradient_loss(x, tok, adv, m, r),
        "KL": lambda m, r: rl.categorical_kl(x, refl, m, r),
        "entropy": lambda m, r: rl.categorical_entropy(x, m, r),
    }
    for name, f in fns.items():
        for r in range(5):
            l = f(none, r)
            assert (l.value == 0).all(), (name, r)
            assert (l.backward() == 0).all(), (name, r)
        per = f(one, rl.NONE).value.cpu().ravel()
        only = per[-2].item()
        assert all(v == 0.0 for i, v in enumerate(per.tolist()) if i != len(per) - 2)
        for r in (rl.TOKEN_MEAN, rl.SEQUENCE_MEAN, rl.SUM):
            assert f(one, r).value.cpu().tolist() == [0.0, only], (name, r)


def test_check_scored_finite_names_the_first_position(oracle):
    """check_scored_finite (src/nn/rl.rs:204-211; its test src/nn/tests/rl.rs:837-846) through the C
    ABI: the same result and message as the oracle's restatement, on the reference's hand cases
    and on random placements of −inf / NaN / +inf under random scoring masks."""
    from noetic_tensor_b200 import ops, rl

    dev = torch.device("cuda:0")
    t = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    lp = [-1.0, -np.inf, -2.0]
    assert rl.check_scored_finite("test", t(lp).reshape(1, 1, 3)) == oracle.check_scored_finite("test", lp)
    assert "position 1" in rl.check_scored_finite("test", t(lp).reshape(1, 1, 3))
    assert rl.check_scored_finite("test", t(lp).reshape(1, 1, 3), t([1.0, 0.0, 1.0]).reshape(1, 1, 3)) is None
    assert rl.check_scored_finite("test", t([-1.0, -3.0, -2.0]).reshape(1, 1, 3)) is None
    g = np.random.default_rng(16)
    for n in (1, 31, 1024, 1025, 70_001):
        for _ in range(6):
            v = -g.uniform(0, 9, n)
            bad = g.choice(n, size=min(n, int(g.integers(0, 4))), replace=False)
            v[bad] = g.choice([-np.inf, np.inf, np.nan], size=bad.size)
            m = (g.uniform(0, 1, n) < 0.6).astype(np.float64) if g.uniform() < 0.7 else None
            got = ops.check_scored_finite("policy_gradient_loss", t(v), None if m is None else t(m))
            assert got == oracle.check_scored_finite("policy_gradient_loss", v.astype(np.float32), m)


def test_losses_refuse_non_finite_scored_log_probs_in_debug_mode(monkeypatch):
    """src/nn/tests/rl.rs:847-855 (debug builds): a scored token the vocabulary mask excludes has
    log-probability −inf and the losses refuse it, naming the position; unscored it passes; with
    the switch off nothing is read back."""
    from noetic_tensor_b200 import rl

    dev = torch.device("cuda:0")
    V = 16
    logits = torch.zeros(1, 1, 2, V, device=dev)
    allow = torch.ones(1, V, dtype=torch.uint8, device=dev)
    allow[0, 5] = 0
    tokens = torch.tensor([[[3, 5]]], dtype=torch.int32, device=dev)
    w = torch.ones(1, 1, device=dev)
    z = rl.Tempered(logits, 1.0, allow)
    monkeypatch.setattr(rl, "DEBUG_CHECKS", True)
    with pytest.raises(RuntimeError, match=r"policy_gradient_loss: the scored log-probability at flat position 1 is -inf \(not finite\)"):
        rl.policy_gradient_loss(z, tokens, w, reduction=rl.SUM)
    skip = torch.tensor([[[1.0, 0.0]]], device=dev)
    rl.policy_gradient_loss(z, tokens, w, mask=skip, reduction=rl.SUM)
    old = torch.tensor([[[-1.0, float("-inf")]]], device=dev)
    ok_tokens = torch.tensor([[[3, 4]]], dtype=torch.int32, device=dev)
    with pytest.raises(RuntimeError, match=r"clipped_policy_loss \(old log-probabilities\): .* position 1 is -inf"):
        rl.clipped_policy_loss(z, ok_tokens, old, w, reduction=rl.SUM)
    with pytest.raises(RuntimeError, match=r"kl_estimate \(reference log-probabilities\): .* position 1 is -inf"):
        rl.kl_estimate(z, ok_tokens, old, rl.K3, reduction=rl.SUM)
    monkeypatch.setattr(rl, "DEBUG_CHECKS", False)
    assert torch.isinf(rl.policy_gradient_loss(z, tokens, w, reduction=rl.SUM).value).all()


@pytest.mark.parametrize("S,B,T", [(2, 3, 4), (3, 5, 7), (8, 32, 1024), (4, 256, 128), (2, 1100, 33), (1, 1, 1)])
def test_token_reduction_bits_do_not_depend_on_the_number_of_gpus(S, B, T):
    """nrl_reduce_tokens equals, to the bit, the two-step form a sharded caller runs
    (nrl_reduce_tokens_partial on each shard's sequences -> pairs concatenated in sequence order ->
    nrl_reduce_tokens_fold) for 1, 2, 3 and 8 shards, and both equal the stated operand order
    evaluated on the host (tests/truth.py). The backward from gathered pairs equals
    nrl_reduce_tokens_bwd on every shard."""
    import truth
    from noetic_tensor_b200 import ops, shard

    dev = torch.device("cuda:0")
    g = np.random.default_rng(S * 1000 + B)
    mask = (g.uniform(0, 1, (S, B, T)) < 0.7).astype(np.float32)
    mask[0, 0] = 0.0
    per = (g.normal(0, 2, (S, B, T)).astype(np.float32)) * mask
    tp, tm = torch.from_numpy(per).to(dev), torch.from_numpy(mask).to(dev)
    host_pairs = truth.warp_seq_pairs(per.reshape(S * B, T), mask.reshape(S * B, T))
    for use_mask in (True, False):
        m = tm if use_mask else None
        hp = host_pairs if use_mask else truth.warp_seq_pairs(per.reshape(S * B, T), None)
        for r in (1, 2, 3, 4):
            whole = ops.reduce_tokens(tp, m, r)
            assert np.array_equal(whole.cpu().numpy().view(np.int32), truth.fold_pairs(hp, S, B, r).view(np.int32)), (r, "vs the stated order")
            up = torch.from_numpy(g.normal(0, 1, tuple(whole.shape)).astype(np.float32)).to(dev)
            d_whole = ops.reduce_tokens_backward((S, B, T), m, r, up).reshape(S * B, T)
            for world in (1, 2, 3, 8):
                pieces = []
                for rank in range(world):
                    b, e = shard.sequence_range(S, B, rank, world)
                    if e > b:
                        pieces.append(ops.reduce_tokens_partial(tp.reshape(S * B, T)[b:e].contiguous(), None if m is None else m.reshape(S * B, T)[b:e].contiguous()))
                pairs = torch.cat(pieces).contiguous()
                assert np.array_equal(pairs.cpu().numpy().view(np.int32), hp.view(np.int32))
                folded = ops.reduce_tokens_fold(pairs, S, B, r)
                assert torch.equal(folded.view(torch.int32), whole.view(torch.int32)), (r, world)
                for rank in range(world):
                    b, e = shard.sequence_range(S, B, rank, world)
                    if e > b:
                        d = ops.reduce_tokens_backward_pairs(r, S, B, T, b, e - b, pairs, None if m is None else m.reshape(S * B, T)[b:e].contiguous(), up)
                        assert torch.equal(d.view(torch.int32), d_whole[b:e].view(torch.int32)), (r, world, rank, "backward")


@pytest.mark.parametrize("S,B,T", [(2, 8, 12), (8, 64, 256), (4, 256, 128), (1, 1100, 33)])
@pytest.mark.parametrize("reduction", [1, 2, 4])
def test_token_objective_equals_the_separate_launches(S, B, T, reduction):
    """nrl_token_objective (one launch) against the eight launches it stands for — token_loss,
    three reduce_tokens, three reduce_tokens_bwd, the backward token_loss — bit for bit: the three
    reduced values and the per-token gradients the row backward takes."""
    from noetic_tensor_b200 import capi, ops

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(S * 100 + B + reduction)
    lp = -torch.rand(S, B, T, generator=g, device=dev) * 6
    old = lp + 0.3 * torch.randn(S, B, T, generator=g, device=dev)
    adv = torch.randn(S, B, generator=g, device=dev)
    kl = torch.rand(S, B, T, generator=g, device=dev)
    ent = torch.rand(S, B, T, generator=g, device=dev) * 5
    mask = (torch.rand(S, B, T, generator=g, device=dev) < 0.7).float()
    mask[0, 0] = 0
    ups = [torch.randn(S, generator=g, device=dev) for _ in range(3)]
    for m in (mask, None):
        for kind, kw in ((capi.LOSS_PPO, dict(other=old, weights=adv, clip_low=0.2, clip_high=0.3, dual=3.0, clamp=20.0)), (capi.LOSS_PG, dict(weights=adv)), (capi.LOSS_K3, dict(other=old, clamp=5.0))):
            o = ops.token_objective(kind, lp, reduction, mask=m, kl=kl, entropy=ent, up_policy=ups[0], up_kl=ups[1], up_entropy=ups[2], **kw)
            per, _ = ops.token_loss(kind, lp, mask=m, want_grad=False, **kw)
            want = [ops.reduce_tokens(per, m, reduction), ops.reduce_tokens(ops.mask_rows(kl, m), m, reduction), ops.reduce_tokens(ops.mask_rows(ent, m), m, reduction)]
            d = [ops.reduce_tokens_backward((S, B, T), m, reduction, u) for u in ups]
            _, g_lp = ops.token_loss(kind, lp, mask=m, upstream=d[0], **kw)
            for got, w, name in zip((o.policy, o.kl, o.entropy, o.g_logp, o.g_kl, o.g_ent), want + [g_lp, d[1], d[2]], ("policy", "kl", "entropy", "g_logp", "g_kl", "g_ent")):
                assert torch.equal(got.view(torch.int32), w.view(torch.int32)), (kind, name, (got - w).abs().max().item())
    with pytest.raises(capi.NrlError):
        ops.token_objective(capi.LOSS_PG, lp, 3, weights=adv)
