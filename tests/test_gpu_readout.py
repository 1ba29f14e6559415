"""The readout-fused statistics (nrl_readout_fwd: tcgen05 product + online-softmax epilogue) through
the C ABI.

The product: the optional bf16 copy of the logits against an f64 product of the same bf16
operands (a bf16 value may land on the neighbouring representable number: f32 accumulation order).
The statistics: with NRL_READOUT_ROUND_BF16 the kernel folds exactly the logits it wrote, so
log-prob, entropy and row statistics are held to the CPU oracle and to nrl_row_fwd on those logits
at the path's tolerance (1e-5 relative or 1e-6 absolute); without rounding they are held to the f64
statistics of the f64 product within 5e-5 relative, the spread an f32-accumulated product of
d = 4096 terms leaves in a logit (the reference's own product, src/tensor/cuda/half_gemm.rs:32-168,
accumulates in f32 in another order). What it replaces: src/nn/decoder.rs:270-279 followed by
src/nn/rl.rs:134-141, 405-414."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def close(got, want, what, rel=1e-5, abs_=1e-6):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want)
    ok = (err <= abs_) | (err <= rel * np.abs(want)) | (got == want)
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} of {ok.size} outside tolerance, worst |Δ| {err.max():.3e}"


def make(rows, d, V, seed):
    g = torch.Generator(device=dev())
    g.manual_seed(seed)
    x = torch.randn(rows, d, generator=g, device=dev()).bfloat16()
    w = (torch.randn(d, V, generator=g, device=dev()) * (3.0 / d ** 0.5)).bfloat16()
    tok = torch.randint(0, V, (rows,), generator=g, device=dev(), dtype=torch.int32)
    return x, w, tok


CASES = [(128, 64, 256), (100, 72, 776), (37, 8, 8), (256, 256, 1024), (1000, 512, 4104), (129, 4096, 32000), (300, 4096, 128256), (2500, 1024, 16384)]


@pytest.mark.parametrize("rows,d,V", CASES)
@pytest.mark.parametrize("layout", ["dV", "Vd"])
def test_readout_statistics_on_the_logits_it_wrote(oracle, rows, d, V, layout):
    from noetic_tensor_b200 import ops

    x, w, tok = make(rows, d, V, rows + V)
    wa = w.t().contiguous() if layout == "Vd" else w
    o = ops.readout_forward(x, wa, tokens=tok, weights_are_vd=(layout == "Vd"), round_bf16=True, want_logits=True)
    assert (o.status == 0).all()
    # the product
    n = min(rows, 160)
    ref = x[:n].double() @ w.double()
    lg = o.logits[:n].double()
    assert ((lg - ref).abs() <= 2.0 ** -7 * ref.abs() + 1e-4).all(), f"logits: worst |Δ| {(lg - ref).abs().max().item():.3e}"
    # the statistics: the oracle on the very logits the kernel folded
    idx = np.random.default_rng(rows).choice(rows, min(rows, 24), replace=False)
    bits = o.logits[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    orc = oracle.sample_inverse_cdf(bits, 1.0, None, given_tokens=tok[idx].cpu().numpy().astype(np.int64))
    close(o.logp[idx].cpu().numpy(), orc["logp"], "logp vs oracle")
    close(o.entropy[idx].cpu().numpy(), orc["entropy"], "entropy vs oracle")
    # and the row kernel on the same logits, every row
    f = ops.row_forward(o.logits, tokens=tok)
    close(o.logp.cpu().numpy(), f.logp.cpu().numpy(), "logp vs nrl_row_fwd")
    close(o.entropy.cpu().numpy(), f.entropy.cpu().numpy(), "entropy vs nrl_row_fwd")
    assert torch.equal(o.rowstats[:, 0], f.rowstats[:, 0]), "the row maximum is exact"
    close(o.rowstats[:, 1].cpu().numpy(), f.rowstats[:, 1].cpu().numpy(), "ln Z vs nrl_row_fwd")
    # run to run, and without the debug output
    again = ops.readout_forward(x, wa, tokens=tok, weights_are_vd=(layout == "Vd"), round_bf16=True)
    for name in ("logp", "entropy", "rowstats"):
        assert torch.equal(getattr(o, name).view(torch.int32), getattr(again, name).view(torch.int32)), name


@pytest.mark.parametrize("rows,d,V", [(256, 256, 1024), (200, 4096, 128256), (1500, 2048, 8192)])
def test_readout_statistics_of_the_f32_accumulators(rows, d, V):
    """Without rounding the logits are the f32 accumulators, as the reference's f32 logits tensor."""
    from noetic_tensor_b200 import ops

    x, w, tok = make(rows, d, V, 7 * rows + V)
    o = ops.readout_forward(x, w, tokens=tok)
    ovd = ops.readout_forward(x, w.t().contiguous(), tokens=tok, weights_are_vd=True)
    n = min(rows, 128)
    ref = x[:n].double() @ w.double()
    lp = torch.log_softmax(ref, 1)
    ent = -(lp.exp() * lp).sum(1)
    lse = torch.logsumexp(ref, 1)
    lpt = lp[torch.arange(n, device=dev()), tok[:n].long()]
    close((o.rowstats[:n, 0].double() + o.rowstats[:n, 1].double()).cpu().numpy(), lse.cpu().numpy(), "m + ln Z", rel=5e-5, abs_=5e-6)
    close(o.entropy[:n].cpu().numpy(), ent.cpu().numpy(), "entropy", rel=5e-5, abs_=5e-6)
    close(o.logp[:n].cpu().numpy(), lpt.cpu().numpy(), "logp", rel=5e-5, abs_=5e-6)
    # the two weight layouts feed the same products in the same order
    for name in ("logp", "entropy", "rowstats"):
        assert torch.equal(getattr(o, name).view(torch.int32), getattr(ovd, name).view(torch.int32)), name


def test_readout_refusals_and_status():
    from noetic_tensor_b200 import capi, ops

    x, w, tok = make(140, 64, 512, 3)
    x[5, 7] = float("nan")
    tok[9] = 512  # no such token
    o = ops.readout_forward(x, w, tokens=tok)
    st = o.status.cpu().numpy()
    assert st[5] == 2 and (np.delete(st, 5) == 0).all()
    assert torch.isnan(o.logp[5]) and torch.isnan(o.entropy[5]) and torch.isnan(o.logp[9]) and torch.isfinite(o.entropy[9])
    with pytest.raises(capi.NrlError):
        ops.readout_forward(x[:, :60].contiguous(), w[:60].contiguous(), tokens=tok)  # d not a multiple of 8
    with pytest.raises(capi.NrlError):
        ops.readout_forward(x, w, tokens=tok, workspace=torch.empty(16, dtype=torch.uint8, device=dev()))


@pytest.mark.parametrize("rows,d,V", [(129, 64, 512), (300, 4096, 128256), (2500, 1024, 16384), (513, 72, 776)])
@pytest.mark.parametrize("layout", ["dV", "Vd"])
def test_readout_cta_pairs_give_the_single_cta_bits(rows, d, V, layout):
    """More than 128 rows run on CTA pairs (tcgen05 cta_group::2: one product over two SMs, each
    loading half of every W tile); NRL_READOUT_ONE_CTA keeps one CTA per 128 rows. The products and
    the fold are the same operations in the same order: the same bits."""
    from noetic_tensor_b200 import ops

    x, w, tok = make(rows, d, V, 11 * rows + V)
    wa = w.t().contiguous() if layout == "Vd" else w
    for rnd in (False, True):
        a = ops.readout_forward(x, wa, tokens=tok, weights_are_vd=(layout == "Vd"), round_bf16=rnd, want_logits=True)
        b = ops.readout_forward(x, wa, tokens=tok, weights_are_vd=(layout == "Vd"), round_bf16=rnd, want_logits=True, one_cta=True)
        assert (a.status == 0).all() and (b.status == 0).all()
        assert torch.equal(a.logits.view(torch.int16), b.logits.view(torch.int16))
        for name in ("logp", "entropy", "rowstats"):
            assert torch.equal(getattr(a, name).view(torch.int32), getattr(b, name).view(torch.int32)), (name, rnd)


@pytest.mark.parametrize("rows,d,V,keep", [(128, 64, 256, None), (100, 72, 776, 0.5), (1000, 512, 4104, 0.1), (300, 4096, 128256, None), (260, 4096, 128256, 0.02), (2500, 1024, 16384, 0.7)])
@pytest.mark.parametrize("layout", ["dV", "Vd"])
def test_readout_sampling_and_masks(oracle, rows, d, V, keep, layout):
    """NRL_READOUT_SAMPLE with and without a byte allow-mask: the tokens against the f64 oracle's
    inverse CDF on the very logits the kernel folded (equal off the CDF boundary rows; the picked
    logit is computed a second time in f32, so a row whose uniform lies within the oracle's
    boundary band may fall either way), never an excluded token, log-prob / entropy within the
    path's tolerance, and nrl_row_fwd's sampler on the same logits, mask and uniforms agreeing."""
    from noetic_tensor_b200 import ops

    x, w, _ = make(rows, d, V, 13 * rows + V)
    wa = w.t().contiguous() if layout == "Vd" else w
    g = torch.Generator(device=dev())
    g.manual_seed(rows)
    u = torch.rand(rows, generator=g, device=dev())
    allow = None
    if keep is not None:
        allow = (torch.rand(rows, V, generator=g, device=dev()) < keep).to(torch.uint8)
        allow[:, V // 3] = 1
    o = ops.readout_forward(x, wa, uniforms=u, allow=allow, weights_are_vd=(layout == "Vd"), round_bf16=True, want_logits=True)
    assert (o.status == 0).all()
    tok = o.tokens.long()
    assert ((tok >= 0) & (tok < V)).all()
    if allow is not None:
        assert allow[torch.arange(rows, device=dev()), tok].all(), "an excluded token was drawn"
    # the row kernel's sampler on the same logits
    f = ops.row_forward(o.logits, allow=allow, uniforms=u)
    differ = (f.tokens != o.tokens)
    # the oracle on a sample of rows (and on every row where the two samplers differ)
    idx = np.unique(np.concatenate([np.random.default_rng(rows).choice(rows, min(rows, 24), replace=False), differ.nonzero().flatten().cpu().numpy()[:40]]))
    bits = o.logits[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    orc = oracle.sample_inverse_cdf(bits, 1.0, u[idx].cpu().numpy(), allow=None if allow is None else allow[idx].cpu().numpy())
    got = o.tokens[idx].cpu().numpy().astype(np.int64)
    bad = (got != orc["tokens"]) & (orc["boundary"] == 0)
    assert not bad.any(), f"{bad.sum()} sampled tokens differ from the oracle off the CDF boundaries"
    same = got == orc["tokens"]
    lp_err = np.abs(o.logp[idx].cpu().numpy()[same] - orc["logp"][same])
    assert ((lp_err <= 1e-6) | (lp_err <= 1e-5 * np.abs(orc["logp"][same])) | (lp_err <= 2.0 ** -7 * 32)).all() and np.count_nonzero(lp_err > 1e-4) <= 2, "logp of drawn tokens vs oracle"
    close(o.entropy[idx].cpu().numpy(), orc["entropy"], "entropy vs oracle")
    agree = ~differ
    # The drawn token's logit is computed a second time (f32 on the CUDA cores); rounded to bf16 it can
    # land on the neighbour of the value the tensor cores' accumulation rounded to: at most a few rows,
    # and never by more than one bf16 step of that logit.
    lp_a, lp_b = o.logp[agree].double(), f.logp[agree].double()
    zt = o.logits[torch.arange(rows, device=dev()), tok][agree].double().abs()
    off = ((lp_a - lp_b).abs() > 1e-6) & ((lp_a - lp_b).abs() > 1e-5 * lp_b.abs())
    assert int(off.sum()) <= max(2, rows // 100) and ((lp_a - lp_b).abs()[off] <= 2.0 ** -7 * zt[off] + 1e-6).all(), "logp vs nrl_row_fwd"
    close(o.entropy.cpu().numpy(), f.entropy.cpu().numpy(), "entropy vs nrl_row_fwd")
    assert int(differ.sum()) <= max(2, rows // 100), f"{int(differ.sum())} of {rows} tokens differ from nrl_row_fwd's sampler"
    # run to run
    again = ops.readout_forward(x, wa, uniforms=u, allow=allow, weights_are_vd=(layout == "Vd"), round_bf16=True)
    assert torch.equal(again.tokens, o.tokens) and torch.equal(again.logp.view(torch.int32), o.logp.view(torch.int32))


@pytest.mark.parametrize("rows,d,V", [(300, 4096, 128256), (1000, 512, 4104)])
def test_readout_sampling_of_the_f32_accumulators(rows, d, V):
    """Without rounding: the drawn tokens' log-probs against the f64 log-softmax of the f64 product at
    those tokens (5e-5 relative: the spread of an f32-accumulated product), and the draw itself
    against the f64 CDF: the token's cumulative interval must contain u·Z up to that spread."""
    from noetic_tensor_b200 import ops

    x, w, _ = make(rows, d, V, 17 * rows + V)
    g = torch.Generator(device=dev())
    g.manual_seed(rows)
    u = torch.rand(rows, generator=g, device=dev())
    o = ops.readout_forward(x, w, uniforms=u)
    n = min(rows, 128)
    ref = x[:n].double() @ w.double()
    lp = torch.log_softmax(ref, 1)
    tok = o.tokens[:n].long()
    # ln Z comes from the tensor cores' accumulation of 4096-term products, the token's logit from an f32
    # FMA chain: the two differ from the exact product by up to ~1e-4 in a logit of magnitude ~10
    close(o.logp[:n].cpu().numpy(), lp[torch.arange(n, device=dev()), tok].cpu().numpy(), "logp of drawn tokens", rel=5e-5, abs_=1e-4)
    cdf = torch.cumsum(lp.exp(), 1)
    hi = cdf[torch.arange(n, device=dev()), tok]
    lo = hi - lp.exp()[torch.arange(n, device=dev()), tok]
    uu = u[:n].double()
    assert ((uu >= lo - 1e-4) & (uu <= hi + 1e-4)).all(), "a drawn token's CDF interval does not hold its uniform"


def test_readout_sampling_distribution_and_refusals():
    """Frequencies over many draws of one small distribution (src/nn/tests/rl.rs:582-629: within 4.5
    standard errors), a row with no allowed token (status 1, token −1) and masks given as [1, V]."""
    from noetic_tensor_b200 import ops

    d, V, draws = 64, 64, 40000
    g = torch.Generator(device=dev())
    g.manual_seed(5)
    h = torch.randn(1, d, generator=g, device=dev()).bfloat16()
    w = (torch.randn(d, V, generator=g, device=dev()) * 0.3).bfloat16()
    x = h.expand(draws, d).contiguous()
    allow = torch.ones(1, V, dtype=torch.uint8, device=dev())
    allow[0, ::5] = 0
    u = torch.rand(draws, generator=g, device=dev())
    o = ops.readout_forward(x, w, uniforms=u, allow=allow)
    z = (h.double() @ w.double())[0]
    z[allow[0] == 0] = float("-inf")
    p = torch.softmax(z, 0).cpu().numpy()
    fr = np.bincount(o.tokens.cpu().numpy(), minlength=V) / draws
    assert (fr[::5] == 0).all()
    assert np.all(np.abs(fr - p) <= 4.5 * np.sqrt(p * (1 - p) / draws) + 1e-12)
    rows_mask = torch.ones(200, V, dtype=torch.uint8, device=dev())
    rows_mask[17] = 0
    o = ops.readout_forward(x[:200].contiguous(), w, uniforms=u[:200].contiguous(), allow=rows_mask)
    st = o.status.cpu().numpy()
    assert st[17] == 1 and o.tokens[17] == -1 and (np.delete(st, 17) == 0).all()


def test_readout_batches_beyond_one_launch():
    """More than 24 576 rows go out as several launches over one workspace (each a whole number of
    waves of CTA pairs): every output row against nrl_row_fwd on the logits the call wrote, given
    tokens and drawn ones, with per-row masks, and against the single launch of NRL_READOUT_ONE_CTA."""
    from noetic_tensor_b200 import capi, ops

    rows, d, V = 60077, 64, 1000
    x, w, tok = make(rows, d, V, 99)
    assert capi.lib().nrl_readout_workspace_bytes(rows, V, d, 0) < capi.lib().nrl_readout_workspace_bytes(rows, V, d, capi.READOUT_ONE_CTA)
    o = ops.readout_forward(x, w, tokens=tok, round_bf16=True, want_logits=True)
    assert (o.status == 0).all()
    f = ops.row_forward(o.logits, tokens=tok)
    close(o.logp.cpu().numpy(), f.logp.cpu().numpy(), "logp vs nrl_row_fwd")
    close(o.entropy.cpu().numpy(), f.entropy.cpu().numpy(), "entropy vs nrl_row_fwd")
    assert torch.equal(o.rowstats[:, 0], f.rowstats[:, 0])
    one = ops.readout_forward(x, w, tokens=tok, round_bf16=True, want_logits=True, one_cta=True)
    assert torch.equal(one.logits.view(torch.int16), o.logits.view(torch.int16))
    close(o.logp.cpu().numpy(), one.logp.cpu().numpy(), "logp vs one launch")
    g = torch.Generator(device=dev())
    g.manual_seed(4)
    u = torch.rand(rows, generator=g, device=dev())
    allow = (torch.rand(rows, V, generator=g, device=dev()) < 0.3).to(torch.uint8)
    allow[:, 5] = 1
    allow[40000] = 0
    s = ops.readout_forward(x, w, uniforms=u, allow=allow, round_bf16=True, want_logits=True)
    st = s.status.cpu().numpy()
    assert st[40000] == 1 and s.tokens[40000] == -1 and (np.delete(st, 40000) == 0).all()
    fs = ops.row_forward(s.logits, allow=allow, uniforms=u)
    keep = torch.ones(rows, dtype=torch.bool, device=dev())
    keep[40000] = False
    differ = (fs.tokens != s.tokens) & keep
    assert int(differ.sum()) <= rows // 100, f"{int(differ.sum())} of {rows} tokens differ from nrl_row_fwd's sampler"
    assert allow[torch.arange(rows, device=dev())[keep], s.tokens.long()[keep]].all()
    close(s.entropy[keep].cpu().numpy(), fs.entropy[keep].cpu().numpy(), "entropy vs nrl_row_fwd")


@pytest.mark.parametrize("rows,d,V,keep", [(300, 4096, 128256, None), (1000, 512, 4104, 0.3), (129, 64, 512, 0.05), (30000, 64, 1000, 0.5)])
@pytest.mark.parametrize("layout", ["dV", "Vd"])
def test_readout_greedy_is_the_first_maximum(rows, d, V, keep, layout):
    """NRL_READOUT_GREEDY (sample_categorical at temperature 0, src/nn/rl.rs:510-529): the first
    maximum of the logits the kernel folded (rounded to bf16 and written, so ties exist and the
    comparison is exact), under an allow-mask too; log-prob = −ln Z at the maximum; a row with
    nothing allowed is refused."""
    from noetic_tensor_b200 import ops

    x, w, _ = make(rows, d, V, 19 * rows + V)
    wa = w.t().contiguous() if layout == "Vd" else w
    allow = None
    if keep is not None:
        g = torch.Generator(device=dev())
        g.manual_seed(V)
        allow = (torch.rand(rows, V, generator=g, device=dev()) < keep).to(torch.uint8)
        allow[:, V // 3] = 1
        allow[11] = 0
    o = ops.readout_forward(x, wa, greedy=True, allow=allow, weights_are_vd=(layout == "Vd"), round_bf16=True, want_logits=True)
    z = o.logits.float()
    if allow is not None:
        z = torch.where(allow.bool(), z, torch.full_like(z, float("-inf")))
    zmax = z.max(dim=1, keepdim=True).values
    first = (z == zmax).float().argmax(dim=1)
    ok = torch.ones(rows, dtype=torch.bool, device=dev())
    if allow is not None:
        ok[11] = False
        assert o.status[11] == 1 and o.tokens[11] == -1
    assert (o.status[ok] == 0).all()
    assert torch.equal(o.tokens.long()[ok], first[ok]), f"{int((o.tokens.long()[ok] != first[ok]).sum())} rows are not the first maximum"
    f = ops.row_forward(o.logits, allow=allow, tokens=o.tokens.clamp_min(0))
    close(o.logp[ok].cpu().numpy(), f.logp[ok].cpu().numpy(), "logp of the maximum vs nrl_row_fwd")
    close(o.logp[ok].cpu().numpy(), (-o.rowstats[ok, 1]).cpu().numpy(), "logp = -ln Z", rel=0, abs_=0)


@pytest.mark.parametrize("tau", [0.7, 1.5])
@pytest.mark.parametrize("rows,d,V,keep", [(300, 4096, 128256, None), (1000, 512, 4104, 0.3)])
def test_readout_temperature(oracle, rows, d, V, keep, tau):
    """logits / τ inside the fused pass (tempered_logits, src/nn/rl.rs:475-486): given tokens,
    sampling and the first maximum against nrl_row_fwd at the same temperature on the (undivided)
    logits the call wrote, and against the oracle on a sample of rows."""
    from noetic_tensor_b200 import ops

    x, w, tok = make(rows, d, V, 23 * rows + V)
    g = torch.Generator(device=dev())
    g.manual_seed(V + rows)
    u = torch.rand(rows, generator=g, device=dev())
    allow = None
    if keep is not None:
        allow = (torch.rand(rows, V, generator=g, device=dev()) < keep).to(torch.uint8)
        allow[:, V // 3] = 1
    o = ops.readout_forward(x, w, tokens=tok, allow=allow, round_bf16=True, want_logits=True, temperature=tau)
    f = ops.row_forward(o.logits, allow=allow, tokens=tok, temperature=tau)
    close(o.logp.cpu().numpy(), f.logp.cpu().numpy(), "logp vs nrl_row_fwd")
    close(o.entropy.cpu().numpy(), f.entropy.cpu().numpy(), "entropy vs nrl_row_fwd")
    assert torch.equal(o.rowstats[:, 0], f.rowstats[:, 0]), "the row maximum is exact"
    idx = np.random.default_rng(rows).choice(rows, 16, replace=False)
    bits = o.logits[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    orc = oracle.sample_inverse_cdf(bits, tau, None, allow=None if allow is None else allow[idx].cpu().numpy(), given_tokens=tok[idx].cpu().numpy().astype(np.int64))
    close(o.entropy[idx].cpu().numpy(), orc["entropy"], "entropy vs oracle")
    lp = o.logp[idx].cpu().numpy()
    finite = np.isfinite(orc["logp"])
    close(lp[finite], orc["logp"][finite], "logp vs oracle")
    s = ops.readout_forward(x, w, uniforms=u, allow=allow, round_bf16=True, want_logits=True, temperature=tau)
    fs = ops.row_forward(s.logits, allow=allow, uniforms=u, temperature=tau)
    assert int((s.tokens != fs.tokens).sum()) <= max(2, rows // 100)
    same = s.tokens == fs.tokens
    d_lp = (s.logp[same] - fs.logp[same]).abs()
    zt = s.logits[torch.arange(rows, device=dev()), s.tokens.long()][same].float().abs()
    assert (d_lp <= 1e-5 * fs.logp[same].abs() + 1e-6 + 2.0 ** -7 * zt / tau).all() and int((d_lp > 1e-4).sum()) <= max(2, rows // 100)
    gr = ops.readout_forward(x, w, greedy=True, allow=allow, round_bf16=True, want_logits=True, temperature=tau)
    fg = ops.row_forward(gr.logits, allow=allow, greedy=True, temperature=tau)
    assert torch.equal(gr.tokens, fg.tokens)
    close(gr.logp.cpu().numpy(), fg.logp.cpu().numpy(), "greedy logp vs nrl_row_fwd")


def test_head_functions_of_the_rl_module():
    """rl.head_token_log_probs / rl.head_sample_categorical (the Python mirrors of Decoder::head
    followed by token_log_probs / sample_categorical): leading shapes, a [1, V] and a per-position
    mask, temperature, temperature 0, and the reference's refusal text; values against the f64
    log-softmax of the f64 product."""
    from noetic_tensor_b200 import rl

    S, B, T, d, V = 2, 3, 20, 64, 512
    g = torch.Generator(device=dev())
    g.manual_seed(3)
    h = torch.randn(S, B, T, d, generator=g, device=dev()).bfloat16()
    w = (torch.randn(d, V, generator=g, device=dev()) * 0.4).bfloat16()
    tok = torch.randint(0, V, (S, B, T), generator=g, device=dev())
    z = h.double() @ w.double()
    lp, ent = rl.head_token_log_probs(h, w, tok)
    want = torch.log_softmax(z, -1)
    assert lp.shape == (S, B, T) and ent.shape == (S, B, T)
    close(lp.cpu().numpy(), want.gather(-1, tok[..., None])[..., 0].cpu().numpy(), "head_token_log_probs", rel=5e-5, abs_=5e-6)
    close(ent.cpu().numpy(), (-(want.exp() * want).sum(-1)).cpu().numpy(), "entropy", rel=5e-5, abs_=5e-6)
    u = torch.rand(S, B, T, generator=g, device=dev())
    shared = torch.ones(1, V, dtype=torch.bool, device=dev())
    shared[0, ::3] = False
    for tau, mask in ((1.0, None), (0.8, shared), (1.3, torch.rand(S, B, T, V, generator=g, device=dev()) < 0.4)):
        if mask is not None and mask.dim() == 4:
            mask[..., 7] = True
        tk, lps, en = rl.head_sample_categorical(h, w, u, vocab_mask=mask, temperature=tau)
        zt = z / tau
        if mask is not None:
            zt = torch.where(mask.expand(S, B, T, V), zt, torch.full_like(zt, float("-inf")))
        p = torch.softmax(zt, -1)
        cdf = p.cumsum(-1)
        hi = cdf.gather(-1, tk.long()[..., None])[..., 0]
        lo = hi - p.gather(-1, tk.long()[..., None])[..., 0]
        assert tk.shape == (S, B, T) and ((u.double() >= lo - 1e-4) & (u.double() <= hi + 1e-4)).all(), tau
        if mask is not None:
            assert mask.expand(S, B, T, V).gather(-1, tk.long()[..., None]).all()
        close(lps.cpu().numpy(), torch.log_softmax(zt, -1).gather(-1, tk.long()[..., None])[..., 0].cpu().numpy(), "log-probs of drawn tokens", rel=5e-5, abs_=1e-4)
        lw = torch.log_softmax(zt, -1)
        close(en.cpu().numpy(), (-(p * torch.where(p > 0, lw, torch.zeros_like(lw))).sum(-1)).cpu().numpy(), "entropy of the tempered distribution", rel=5e-5, abs_=5e-6)
    # scoring under the mask and temperature the tokens were drawn with gives the sampler's log-probs
    tk_s, lp_s, en_s = rl.head_sample_categorical(h, w, u, vocab_mask=shared, temperature=0.8)
    lp_g, en_g = rl.head_token_log_probs(h, w, tk_s, vocab_mask=shared, temperature=0.8)
    close(lp_g.cpu().numpy(), lp_s.cpu().numpy(), "scored vs sampled log-probs", rel=1e-5, abs_=1e-4)
    assert torch.equal(en_g.view(torch.int32), en_s.view(torch.int32))
    # the shared mask as int32 words of bits: the byte mask's draws
    words = torch.from_numpy(np.packbits(shared.cpu().numpy().astype(np.uint8), axis=1, bitorder="little").view(np.int32)).to(dev())
    tb, lb, eb = rl.head_sample_categorical(h, w, u, vocab_mask=words, temperature=0.8)
    ta, la, ea = rl.head_sample_categorical(h, w, u, vocab_mask=shared, temperature=0.8)
    assert torch.equal(ta, tb) and torch.equal(la.view(torch.int32), lb.view(torch.int32)) and torch.equal(ea.view(torch.int32), eb.view(torch.int32))
    tk0, lp0, _ = rl.head_sample_categorical(h, w, None, vocab_mask=shared)
    z0 = torch.where(shared.expand(S, B, T, V), z, torch.full_like(z, float("-inf")))
    assert ((z0.max(-1).values - z0.gather(-1, tk0.long()[..., None])[..., 0]) <= 1e-4).all()
    none = torch.ones(S, B, T, V, dtype=torch.bool, device=dev())
    none[0, 0, 5] = False
    with pytest.raises(RuntimeError, match="position 5 has no allowed token"):
        rl.head_sample_categorical(h, w, u, vocab_mask=none)


@pytest.mark.parametrize("rows,d,V", [(300, 4096, 128256), (1000, 512, 4104), (30000, 64, 1000)])
def test_readout_bit_packed_masks(rows, d, V):
    """NRL_READOUT_MASK_BITS: the allow-mask as one bit per token (what grammar engines emit), per row
    and shared by all rows, padded word counts too: the byte mask's results bit for bit, for given
    tokens, sampling and the first maximum."""
    from noetic_tensor_b200 import ops

    x, w, tok = make(rows, d, V, 29 * rows + V)
    g = torch.Generator(device=dev())
    g.manual_seed(rows + V)
    u = torch.rand(rows, generator=g, device=dev())
    for shared in (False, True):
        n = 1 if shared else rows
        allow = (torch.rand(n, V, generator=g, device=dev()) < 0.2).to(torch.uint8)
        allow[:, V // 3] = 1
        words = (V + 31) // 32 + (3 if shared else 0)  # a padded row stride is allowed
        packed = np.packbits(np.pad(allow.cpu().numpy(), ((0, 0), (0, words * 32 - V))), axis=1, bitorder="little").view(np.int32)
        bits = torch.from_numpy(packed).to(dev()).contiguous()
        for kw in (dict(tokens=tok), dict(uniforms=u), dict(greedy=True)):
            a = ops.readout_forward(x, w, allow=allow, temperature=0.9, **kw)
            b = ops.readout_forward(x, w, allow_bits=bits, temperature=0.9, **kw)
            assert torch.equal(a.status, b.status) and (a.status == 0).all()
            if a.tokens is not None:
                assert torch.equal(a.tokens, b.tokens), kw.keys()
            for name in ("logp", "entropy", "rowstats"):
                assert torch.equal(getattr(a, name).view(torch.int32), getattr(b, name).view(torch.int32)), (name, list(kw))
    with pytest.raises(Exception):
        ops.readout_forward(x, w, tokens=tok, allow_bits=bits[:, :2].contiguous())
