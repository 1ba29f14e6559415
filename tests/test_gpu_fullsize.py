"""The benchmark's own shapes on the GPU: full vocabulary rows of configurations 3, 4 and 5 in
batches of several GB (far beyond what the CPU oracle can finish), checked through properties
that do not depend on size, plus the oracle on a random sample of the rows.

Properties: sampled tokens are allowed ones; log-probs ≤ 0; 0 ≤ entropy ≤ ln(#allowed); KL ≥ 0
up to rounding; every row of d(logits) sums to ~0 (softmax gradients), is exactly zero where the
mask excludes the token and exactly zero on unscored rows; two runs are bitwise identical.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _check_sample(oracle, f, x, r, m, u, idx, V):
    """The oracle on rows `idx`: tokens equal off the CDF boundaries, values within tolerance."""
    xi, ri = _bits(x[idx]), (None if r is None else _bits(r[idx]))
    mi = None if m is None else m[idx].cpu().numpy()
    o = oracle.sample_inverse_cdf(xi, 1.0, u[idx].cpu().numpy(), ref_logits=ri, allow=mi)
    tok = f.tokens[idx].cpu().numpy().astype(np.int64)
    differ = tok != o["tokens"]
    assert not (differ & (o["boundary"] == 0)).any(), f"{(differ & (o['boundary'] == 0)).sum()} tokens differ off the CDF boundaries"

    def close(a, b, what):
        a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
        ok = (np.abs(a - b) <= 1e-6) | (np.abs(a - b) <= 1e-5 * np.abs(b))
        assert ok.all(), f"{what}: worst |Δ| {np.abs(a - b).max():.3e}"

    same = ~differ
    close(f.logp[idx].cpu().numpy()[same], o["logp"][same], "logp")
    close(f.entropy[idx].cpu().numpy(), o["entropy"], "entropy")
    if r is not None:
        close(f.kl[idx].cpu().numpy(), o["kl"], "kl")
    return int(differ.sum()), int(o["boundary"].sum())


def _check_grad_sample(oracle, d, x, r, m, tokens, idx, V, g_lp, g_kl, g_ent):
    """d(logits) of rows `idx` against the oracle's tape (f64 to 2e-6, f32 to the reference's
    device tolerance 1e-4 of |Δ|/(1+|ref|), src/nn/tests/gpu/rl.rs:106-123), with the rows' allow
    mask as the full additive −inf vocabulary mask."""
    n = idx.numel()
    xi, ri = _bits(x[idx]), (None if r is None else _bits(r[idx]))
    vm = None if m is None else np.where(m[idx].cpu().numpy() != 0, 0.0, -np.inf)
    tok = tokens[idx].cpu().numpy().astype(np.int64)
    up = lambda g: g[idx].cpu().numpy().astype(np.float64)
    got = d[idx].cpu().numpy().astype(np.float64).ravel()
    shape = (1, 1, n, V)
    for dt, tol in ((oracle.F64, 2e-6), (oracle.F32, 1e-4)):
        want = np.zeros(n * V)
        if g_lp is not None:
            want += oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, shape, dtype=dt, logits=xi, tokens=tok, vocab_mask=vm, upstream=up(g_lp))[1]
        if g_ent is not None:
            want += oracle.rl_eval(oracle.OP_ENTROPY, shape, dtype=dt, logits=xi, vocab_mask=vm, upstream=up(g_ent))[1]
        if g_kl is not None:
            want += oracle.rl_eval(oracle.OP_REFERENCE_KL, shape, dtype=dt, logits=xi, ref_logits=ri, vocab_mask=vm, upstream=up(g_kl))[1]
        err = np.abs(got - want) / (1.0 + np.abs(want))
        assert np.nanmax(err) <= tol and not np.isnan(got).any(), f"d(logits) vs oracle dtype {dt}: {np.nanmax(err):.3e}"


def _properties(f, m, rows, V):
    tok = f.tokens.long()
    assert (f.status == 0).all()
    assert ((tok >= 0) & (tok < V)).all()
    if m is not None:
        assert m[torch.arange(rows, device=m.device), tok].all(), "an excluded token was drawn"
        allowed = m.sum(dim=1).float()
    else:
        allowed = torch.full((rows,), float(V), device=tok.device)
    assert (f.logp <= 1e-6).all() and torch.isfinite(f.logp).all()
    assert (f.entropy >= -1e-5).all() and (f.entropy <= torch.log(allowed) + 1e-4).all()
    if f.kl is not None:
        assert (f.kl >= -1e-5).all() and torch.isfinite(f.kl).all()


def test_config3_headline_rows(oracle):
    """bf16 logits ~N(0,3) + log-Zipf prior, U8 grammar masks, bf16 reference: 8192 full rows."""
    from noetic_tensor_b200 import ops, synth

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    rows, V = 8192, 128256
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev, bias=synth.zipf_bias(V, 1.1, gen, dev))
    r = synth.perturbed(x, 0.05, gen)
    m = synth.grammar_masks(rows, V, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    _properties(f, m, rows, V)
    g = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    for name in ("tokens", "logp", "ref_logp", "kl", "entropy", "rowstats"):
        a, b = getattr(f, name), getattr(g, name)
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a, b.view(torch.int32) if b.dtype == torch.float32 else b), name
    idx = torch.from_numpy(np.random.default_rng(0).choice(rows, 96, replace=False)).to(dev)
    n_diff, n_bnd = _check_sample(oracle, f, x, r, m, u, idx, V)
    print(f"config 3: {n_diff} of 96 sampled rows differ from the f64 oracle, all among its {n_bnd} boundary rows")
    # backward: scored and unscored rows
    score = (torch.rand(rows, generator=gen, device=dev) < 0.75).float()
    d = ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=score, g_kl=0.04 * score, g_ent=-0.01 * score)
    assert torch.isfinite(d).all()
    assert (d[score == 0] == 0).all(), "an unscored row has a gradient"
    assert (d[m == 0] == 0).all(), "an excluded token has a gradient"
    assert d.sum(dim=1).abs().max().item() < 2e-3
    _check_grad_sample(oracle, d, x, r, m, f.tokens, idx[:8], V, score, 0.04 * score, -0.01 * score)


def test_config4_ppo_rows(oracle):
    """bf16 logits ~N(0,2.5) at V = 151936 with a reference, no mask: 4096 full rows."""
    from noetic_tensor_b200 import ops, synth

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    rows, V = 4096, 151936
    x = synth.normal_logits(rows, V, 2.5, torch.bfloat16, gen, dev)
    r = synth.perturbed(x, 0.05, gen)
    u = synth.uniforms(rows, gen, dev)
    f = ops.row_forward(x, ref_logits=r, uniforms=u)
    _properties(f, None, rows, V)
    assert torch.equal(f.tokens, ops.row_forward(x, ref_logits=r, uniforms=u).tokens)
    idx = torch.from_numpy(np.random.default_rng(1).choice(rows, 48, replace=False)).to(dev)
    n_diff, n_bnd = _check_sample(oracle, f, x, r, None, u, idx, V)
    print(f"config 4: {n_diff} of 48 sampled rows differ from the f64 oracle, all among its {n_bnd} boundary rows")
    ones = torch.ones(rows, device=dev)
    d = ops.row_backward(x, f, ref_logits=r, g_logp=ones, g_kl=0.04 * ones, g_ent=-0.01 * ones)
    assert torch.isfinite(d).all() and d.sum(dim=1).abs().max().item() < 2e-3
    _check_grad_sample(oracle, d, x, r, None, f.tokens, idx[:6], V, ones, 0.04 * ones, -0.01 * ones)
    # the sampled token's entry is the only positive one of the log-prob term
    d1 = ops.row_backward(x, f, g_logp=ones)
    picked = d1[torch.arange(rows, device=dev), f.tokens.long()]
    assert torch.allclose(picked, 1 - torch.exp(f.logp), atol=2e-6)


def test_config5_sparse_rows(oracle):
    """bf16 logits ~N(0,4) at V = 262144, 1–8 allowed tokens per row shifted 30 below the maximum."""
    from noetic_tensor_b200 import ops, synth

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    rows, V = 2048, 262144
    x = synth.normal_logits(rows, V, 4.0, torch.bfloat16, gen, dev)
    m, idx8 = synth.sparse_masks(rows, V, gen, dev)
    live = idx8 >= 0
    rr = torch.arange(rows, device=dev)[:, None].expand(rows, 8)
    x[rr[live], idx8[live]] -= 30.0
    r = synth.perturbed(x, 0.1, gen)
    u = synth.uniforms(rows, gen, dev)
    f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    _properties(f, m, rows, V)
    one = m.sum(dim=1) == 1
    assert one.any() and (f.entropy[one].abs() < 1e-6).all() and (f.logp[one].abs() < 1e-6).all(), "a single allowed token has probability 1"
    idx = torch.from_numpy(np.random.default_rng(2).choice(rows, 32, replace=False)).to(dev)
    _check_sample(oracle, f, x, r, m, u, idx, V)
    ones = torch.ones(rows, device=dev)
    d = ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=ones, g_kl=ones)
    assert (d[m == 0] == 0).all() and torch.isfinite(d).all()
    _check_grad_sample(oracle, d, x, r, m, f.tokens, idx[:4], V, ones, ones, None)
