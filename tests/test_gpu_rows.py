"""GPU parity of the row kernels (nrl_row_fwd / nrl_row_bwd) against the CPU oracle, through the
C ABI. Tolerances are the target's: 1e-5 relative or 1e-6 absolute in f32; sampled tokens must be
identical except on boundary rows (u·Z within 1e-6·Z of a CDF step), which are counted."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

INF = float("inf")


def dev():
    return torch.device("cuda:0")


def to_dev(a, dtype):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
    return t.to(dtype) if dtype is not None else t


def stored(logits_f32, dtype):
    """(device tensor, host array as the oracle takes it) for f32 or bf16 storage."""
    t = torch.from_numpy(logits_f32.astype(np.float32)).to(dev()).to(dtype)
    if dtype == torch.bfloat16:
        host = t.view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        host = t.cpu().numpy()
    return t, host


def assert_close(got, want, what, rel=1e-5, abs_=1e-6):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    same = (got == want) | (np.isnan(got) & np.isnan(want))
    err = np.abs(got - want)
    ok = same | (err <= abs_) | (err <= rel * np.abs(want))
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} of {ok.size} outside 1e-5 rel / 1e-6 abs; worst |Δ| {np.nanmax(np.where(same, 0, err)):.3e}"


def run_case(oracle, rows, V, dtype, *, ref, allow_kind, add, tau, seed, scale=2.0, check_bwd=True):
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(seed)
    x = g.normal(0, scale, (rows, V)).astype(np.float32)
    xt, xh = stored(x, dtype)
    rt = rh = None
    if ref:
        r = (x + g.normal(0, 0.1, (rows, V))).astype(np.float32)
        rt, rh = stored(r, dtype)
    allow = None
    if allow_kind:
        n = 1 if allow_kind == "broadcast" else rows
        allow = (g.uniform(0, 1, (n, V)) < 0.75).astype(np.uint8)
        allow[:, 0] = 1
    addm = None
    if add:
        addm = np.where(g.uniform(0, 1, (1, V)) < 0.2, -INF if add == "inf" else -1e9, 0.0).astype(np.float32)
        addm[:, 0] = 0.0
    u = oracle.row_uniforms(seed, "uniforms", rows)
    kw = dict(ref_logits=rt, allow=None if allow is None else to_dev(allow, None), add_mask=None if addm is None else to_dev(addm, None), temperature=tau)
    f = ops.row_forward(xt, uniforms=to_dev(u, None), **kw)
    o = oracle.sample_inverse_cdf(xh, tau, u, ref_logits=rh, add_mask=addm, allow=allow)
    tok = f.tokens.cpu().numpy().astype(np.int64)
    assert (f.status.cpu().numpy() == o["status"]).all()
    differ = tok != o["tokens"]
    assert not (differ & (o["boundary"] == 0)).any(), f"{np.count_nonzero(differ & (o['boundary'] == 0))} sampled tokens differ off the CDF boundaries"
    if allow is not None:
        al = np.broadcast_to(allow, (rows, V))
        assert al[np.arange(rows), tok].all(), "an excluded token was drawn"
    # values for the oracle's tokens: re-run with the tokens given so boundary rows compare too
    f2 = ops.row_forward(xt, tokens=to_dev(o["tokens"].astype(np.int32), None), **kw)
    assert_close(f2.logp.cpu().numpy(), o["logp"], "logp")
    assert_close(f2.entropy.cpu().numpy(), o["entropy"], "entropy")
    same = ~differ
    assert_close(f.logp.cpu().numpy()[same], o["logp"][same], "logp of sampled tokens")
    if ref:
        assert_close(f2.kl.cpu().numpy(), o["kl"], "kl")
        assert_close(f2.ref_logp.cpu().numpy(), o["ref_logp"], "ref_logp")
    # greedy: first maximum, exact
    fg = ops.row_forward(xt, greedy=True, **kw)
    og = oracle.sample_inverse_cdf(xh, 0.0, None, add_mask=None if addm is None else addm, allow=allow)
    if tau == 1.0:
        assert np.array_equal(fg.tokens.cpu().numpy().astype(np.int64), og["tokens"])
    # bitwise run to run
    f3 = ops.row_forward(xt, uniforms=to_dev(u, None), **kw)
    for name in ("tokens", "logp", "entropy", "kl", "rowstats"):
        a, b = getattr(f, name), getattr(f3, name)
        if a is not None:
            assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a, b.view(torch.int32) if b.dtype == torch.float32 else b), name
    if not check_bwd:
        return
    # backward against the f32 CpuRef restatement and the f64 path
    S, B, T = 1, 1, rows
    glp, gkl, gen = (g.uniform(-1, 1, rows).astype(np.float32) for _ in range(3))
    d = ops.row_backward(xt, f2, g_logp=to_dev(glp, None), g_kl=to_dev(gkl, None) if ref else None, g_ent=to_dev(gen, None), **kw).cpu().numpy().astype(np.float64)
    # the reference's vocabulary mask is additive and broadcasts at the logits' rank (src/nn/rl.rs:475-486):
    # a per-row allow-mask is the full [1,1,rows,V] additive mask with -inf at excluded tokens
    vm = None
    if addm is not None or allow is not None:
        per_row = allow is not None and allow.shape[0] != 1
        vm = np.zeros((rows, V) if per_row else V)
        if addm is not None:
            vm = vm + addm[0]
        if allow is not None:
            vm = np.where((allow if per_row else allow[0]) != 0, vm, -INF)
    for dt, tol in ((oracle.F64, 2e-6), (oracle.F32, 1e-4)):
        want = np.zeros(rows * V)
        _, g1 = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, (S, B, T, V), dtype=dt, logits=xh, tokens=o["tokens"], vocab_mask=vm, temperature=tau, upstream=glp)
        want += g1
        _, g3 = oracle.rl_eval(oracle.OP_ENTROPY, (S, B, T, V), dtype=dt, logits=xh, vocab_mask=vm, temperature=tau, upstream=gen)
        want += g3
        if ref:
            _, g2 = oracle.rl_eval(oracle.OP_REFERENCE_KL, (S, B, T, V), dtype=dt, logits=xh, ref_logits=rh, vocab_mask=vm, temperature=tau, upstream=gkl)
            want += g2
        err = np.abs(d.ravel() - want) / (1.0 + np.abs(want))
        assert np.nanmax(err) <= tol, f"d(logits) vs oracle dtype {dt}: {np.nanmax(err):.3e}"


@pytest.mark.parametrize("V", [1, 2, 7, 8, 9, 16, 33, 255, 256, 257, 1023, 1024, 1025, 4104, 32000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shapes_plain(oracle, V, dtype):
    run_case(oracle, 37, V, dtype, ref=False, allow_kind=None, add=None, tau=1.0, seed=V)


@pytest.mark.parametrize("V", [5, 24, 264, 1000, 8192])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("allow_kind", [None, "rows", "broadcast"])
def test_shapes_with_reference_and_masks(oracle, V, dtype, allow_kind):
    run_case(oracle, 29, V, dtype, ref=True, allow_kind=allow_kind, add=None, tau=1.0, seed=100 + V)


@pytest.mark.parametrize("V", [24, 1000, 4096])
@pytest.mark.parametrize("add", ["inf", "1e9"])
@pytest.mark.parametrize("tau", [0.7, 1.0, 1.7])
def test_temperature_and_additive_mask(oracle, V, add, tau):
    run_case(oracle, 19, V, torch.float32, ref=True, allow_kind=None, add=add, tau=tau, seed=200 + V)


def test_config1_toy(oracle):
    # logits [4,2,8,16] f32 ~ N(0,1), keep-prob 0.75 mask with token 0 always allowed, one uniform per row
    run_case(oracle, 4 * 2 * 8, 16, torch.float32, ref=True, allow_kind="rows", add=None, tau=1.0, seed=1, scale=1.0)


@pytest.mark.parametrize("rows,V,dtype", [(8, 128256, torch.bfloat16), (3, 32000, torch.float32), (40, 151936, torch.bfloat16), (2, 262144, torch.bfloat16)])
def test_split_rows_use_scratch(oracle, rows, V, dtype):
    from noetic_tensor_b200 import capi

    assert capi.lib().nrl_row_fwd_workspace_bytes(rows, V) > 0
    run_case(oracle, rows, V, dtype, ref=True, allow_kind="rows", add=None, tau=1.0, seed=300 + rows, scale=3.0, check_bwd=False)


def test_large_vocab_fused_rows(oracle):
    # enough rows for the one-block-per-row kernel at the Llama-3 vocabulary
    run_case(oracle, 300, 128256, torch.bfloat16, ref=True, allow_kind="rows", add=None, tau=1.0, seed=7, scale=3.0, check_bwd=False)


def test_peaked_rows_and_sparse_masks(oracle):
    """Rows that allow 1–8 tokens far below the row maximum (the extreme-sparse-mask config)."""
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(5)
    rows, V = 64, 262144
    x = g.normal(0, 4, (rows, V)).astype(np.float32)
    allow = np.zeros((rows, V), dtype=np.uint8)
    for r in range(rows):
        k = 1 if r % 10 == 0 else int(g.integers(1, 9))
        idx = g.choice(V, k, replace=False)
        allow[r, idx] = 1
        x[r, idx] -= 30.0
    ref = (x + g.normal(0, 0.1, (rows, V))).astype(np.float32)
    xt, xh = stored(x, torch.bfloat16)
    rt, rh = stored(ref, torch.bfloat16)
    u = oracle.row_uniforms(9, "sparse", rows)
    f = ops.row_forward(xt, ref_logits=rt, allow=to_dev(allow, None), uniforms=to_dev(u, None))
    o = oracle.sample_inverse_cdf(xh, 1.0, u, ref_logits=rh, allow=allow)
    tok = f.tokens.cpu().numpy().astype(np.int64)
    assert not ((tok != o["tokens"]) & (o["boundary"] == 0)).any()
    assert allow[np.arange(rows), tok].all()
    same = tok == o["tokens"]
    assert_close(f.logp.cpu().numpy()[same], o["logp"][same], "logp")
    assert_close(f.kl.cpu().numpy(), o["kl"], "kl")
    assert_close(f.entropy.cpu().numpy(), o["entropy"], "entropy")


def test_refused_rows(oracle):
    """No allowed token or a NaN: status set, token −1, the reference's panic text from the host check."""
    from noetic_tensor_b200 import ops

    V = 48
    x = np.zeros((4, V), dtype=np.float32)
    allow = np.ones((4, V), dtype=np.uint8)
    allow[1] = 0
    x[2, 5] = np.nan
    x[3] = -INF
    f = ops.row_forward(to_dev(x, None), allow=to_dev(allow, None), uniforms=to_dev(np.full(4, 0.5, np.float32), None))
    assert f.status.cpu().tolist() == [0, 1, 2, 1]
    assert f.tokens.cpu().tolist()[1:] == [-1, -1, -1]
    assert 0 <= f.tokens.cpu().tolist()[0] < V
    with pytest.raises(RuntimeError, match="position 1 has no allowed token"):
        ops.check_status(f.status)
    # additive −inf everywhere is the same refusal (src/nn/tests/rl.rs:631-637)
    add = np.array([[0.0] * V, [-INF] * V], dtype=np.float32)
    f = ops.row_forward(to_dev(np.zeros((2, V), np.float32), None), add_mask=to_dev(add, None), uniforms=to_dev(np.full(2, 0.5, np.float32), None))
    assert f.status.cpu().tolist() == [0, 1]


def test_sampler_distribution_and_reproducibility(oracle):
    """The reference sampler test's shape (src/nn/tests/gpu/rl.rs:157-174): [4·128, 96] logits with
    every seventh token excluded; tokens equal the f64 oracle's off the CDF boundaries, none
    excluded, greedy exactly the oracle's, identical run to run. Frequencies over 40 000 draws
    within 4.5 standard errors (src/nn/tests/rl.rs:582-629)."""
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(960)
    n, V = 4 * 128, 96
    x = g.uniform(-3, 3, (n, V)).astype(np.float32)
    addm = np.where(np.arange(V) % 7 == 3, -INF, 0.0).astype(np.float32)[None]
    xt = to_dev(x, None)
    for tau, root in ((1.0, 11), (0.7, 12)):
        u = oracle.row_uniforms(root, "device sampler", n)
        f = ops.row_forward(xt, add_mask=to_dev(addm, None), temperature=tau, uniforms=to_dev(u, None))
        o = oracle.sample_inverse_cdf(x, tau, u, add_mask=addm)
        tok = f.tokens.cpu().numpy().astype(np.int64)
        assert (tok % 7 != 3).all()
        assert not ((tok != o["tokens"]) & (o["boundary"] == 0)).any()
        assert torch.equal(f.tokens, ops.row_forward(xt, add_mask=to_dev(addm, None), temperature=tau, uniforms=to_dev(u, None)).tokens)
    fg = ops.row_forward(xt, add_mask=to_dev(addm, None), greedy=True)
    assert np.array_equal(fg.tokens.cpu().numpy(), oracle.sample_inverse_cdf(x, 0.0, None, add_mask=addm)["tokens"])
    # frequencies
    v, draws = 6, 40_000
    row = np.array([0.4, -1.0, 1.2, 3.0, 0.0, -0.3], dtype=np.float32)
    mrow = np.array([[0.0, 0.0, 0.0, -INF, 0.5, 0.0]], dtype=np.float32)
    u = oracle.row_uniforms(5, "sampler test", draws)
    f = ops.row_forward(to_dev(np.tile(row, (draws, 1)), None), add_mask=to_dev(mrow, None), temperature=0.7, uniforms=to_dev(u, None))
    z = row.astype(np.float64) / np.float32(0.7) + mrow[0]
    p = np.exp(z - z.max())
    p /= p.sum()
    fr = np.bincount(f.tokens.cpu().numpy(), minlength=v) / draws
    assert fr[3] == 0
    assert np.all(np.abs(fr - p) <= 4.5 * np.sqrt(p * (1 - p) / draws) + 1e-12)


@pytest.mark.parametrize("V,dtype,masked", [(1000, torch.float32, False), (4104, torch.bfloat16, True), (37, torch.bfloat16, False), (128256, torch.bfloat16, True)])
def test_backward_accumulate_adds_into_d_logits(V, dtype, masked):
    """Three separate backward calls adding into one d(logits) (what a tape does with three nodes
    on the same logits) equal the single combined call to rounding, keep unscored rows and
    excluded entries exactly as they were, and `accumulate` on a pre-filled buffer adds to it."""
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(V)
    rows = 24
    x, _ = stored(g.normal(0, 2, (rows, V)), dtype)
    r, _ = stored(g.normal(0, 2, (rows, V)), dtype)
    m = None
    if masked:
        mm = (g.uniform(0, 1, (rows, V // 8)) < 0.5).repeat(8, axis=1)  # whole excluded vectors, as a grammar mask has
        mm = np.concatenate([mm, np.ones((rows, V - mm.shape[1]), bool)], axis=1) & (g.uniform(0, 1, (rows, V)) < 0.9)
        mm[:, 0] = True
        m = to_dev(mm.astype(np.uint8), None)
    f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=to_dev(g.uniform(0, 1, rows).astype(np.float32), None))
    score = to_dev((np.arange(rows) % 4 != 1).astype(np.float32), None)
    glp, gkl, gen = score * 0.7, score * 0.04, score * -0.01
    whole = ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=glp, g_kl=gkl, g_ent=gen)
    d = ops.row_backward(x, f, allow=m, g_logp=glp)
    base = d.clone()
    assert ops.row_backward(x, f, ref_logits=r, allow=m, g_kl=gkl, out=d, accumulate=True) is d
    ops.row_backward(x, f, allow=m, g_ent=gen, out=d, accumulate=True)
    err = (d - whole).abs()
    assert (err <= 1e-6 + 1e-5 * whole.abs()).all(), err.max().item()
    assert not torch.equal(d, base)
    assert (d[score == 0] == 0).all()
    if m is not None:
        assert (d[m == 0] == 0).all()
    # adding onto a buffer that holds something else: rows with zero upstream keep it bit for bit
    pre = torch.full_like(whole, 0.25)
    ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=glp, g_kl=gkl, g_ent=gen, out=pre, accumulate=True)
    assert torch.equal(pre[score == 0], torch.full_like(pre[score == 0], 0.25))
    assert ((pre - 0.25 - whole).abs() <= 1e-6 + 1e-5 * whole.abs()).all()


@pytest.mark.parametrize("rows,V,keep,ref,dtype", [
    (2400, 4104, 0.05, True, torch.bfloat16), (2400, 32000, 0.75, True, torch.bfloat16), (1500, 128256, 0.02, True, torch.bfloat16),
    (1300, 128256, 0.6, False, torch.bfloat16), (4096, 1000, 0.3, True, torch.bfloat16), (1300, 32000, 0.2, True, torch.float32),
    (2400, 32000, None, True, torch.bfloat16), (1300, 128256, None, False, torch.bfloat16), (1300, 32000, None, False, torch.float32),
    (4096, 1000, None, True, torch.float32), (1200, 151936, None, True, torch.bfloat16)])
def test_grouped_forward_equals_the_per_row_kernel(oracle, rows, V, keep, ref, dtype):
    """Many byte-masked rows take the grouped kernel (a block owns a few rows, its warps take
    (row, part) tickets, a row's tail overlaps the next rows' streaming). Its per-row statistics
    must equal the one-block-per-row kernel's within the tolerance (it splits rows finer); sampled
    tokens may differ only on CDF boundary rows; the densest masks overflow the per-part log and
    take the scan fallback."""
    from noetic_tensor_b200 import ops

    g = torch.Generator(device=dev())
    g.manual_seed(rows + V)
    x = (torch.randn(rows, V, generator=g, device=dev()) * 2.5).to(dtype)
    r = (x.float() + 0.1 * torch.randn(rows, V, generator=g, device=dev())).to(dtype) if ref else None
    m = None
    if keep is not None:
        m = (torch.rand(rows, V, generator=g, device=dev()) < keep).to(torch.uint8)
        m[:, V // 2] = 1
        m[7] = 0  # a row with no allowed token
    else:
        x[7] = float("-inf")  # the same without a mask
    u = torch.rand(rows, generator=g, device=dev())
    runs = {}
    for mode in ("1", "0"):
        kw = dict(row_per_block=(mode == "0"))
        runs[mode] = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u, **kw)
        again = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u, **kw)
        given = ops.row_forward(x, ref_logits=r, allow=m, tokens=runs[mode].tokens.clamp_min(0), **kw)
        assert torch.equal(again.tokens, runs[mode].tokens) and torch.equal(again.logp.view(torch.int32), runs[mode].logp.view(torch.int32))
        ok = runs[mode].status == 0
        assert torch.equal(given.logp.view(torch.int32)[ok], runs[mode].logp.view(torch.int32)[ok]), "log-prob of the given token differs from the sampled one's"
    a, b = runs["1"], runs["0"]
    assert a.status.cpu().tolist() == b.status.cpu().tolist() and a.status[7] == 1 and a.tokens[7] == -1
    okr = (a.status == 0).cpu().numpy()
    for name in ("rowstats", "entropy", "logp") + (("kl",) if ref else ()):
        ga, gb = getattr(a, name).cpu().numpy()[okr], getattr(b, name).cpu().numpy()[okr]
        if name == "logp":
            same_tok = (a.tokens == b.tokens).cpu().numpy()[okr]
            ga, gb = ga[same_tok], gb[same_tok]
        assert_close(ga, gb, name)  # the two kernels split a row into parts differently: equal to rounding
    differ = (a.tokens != b.tokens).nonzero().flatten()
    idx = torch.unique(torch.cat([differ, torch.arange(0, rows, max(1, rows // 48), device=dev())]))
    idx = idx[idx != 7]
    xi = x[idx].view(torch.int16).cpu().numpy().view(np.uint16) if dtype == torch.bfloat16 else x[idx].cpu().numpy()
    o = oracle.sample_inverse_cdf(xi, 1.0, u[idx].cpu().numpy(), allow=None if m is None else m[idx].cpu().numpy())
    for f in (a, b):
        tok = f.tokens[idx].cpu().numpy().astype(np.int64)
        bad = (tok != o["tokens"]) & (o["boundary"] == 0)
        assert not bad.any(), f"{bad.sum()} tokens differ from the oracle off the CDF boundaries"
        same = tok == o["tokens"]
        assert_close(f.logp[idx].cpu().numpy()[same], o["logp"][same], "logp")
    # (every differing row was checked above to be one of the oracle's boundary rows)
    assert len(differ) <= max(4, rows // 50), f"{len(differ)} rows differ between the two kernels"


def _grammar_mask_np(g, rows, V):
    """1–4 contiguous allowed bands of width 64–4096 (clipped to V) plus 1 % random tokens: most
    8-token vectors of a row are excluded whole, some hold one allowed token."""
    m = g.uniform(0, 1, (rows, V)) < 0.01
    for r in range(rows):
        for _ in range(int(g.integers(1, 5))):
            w = int(g.integers(64, min(4096, V) + 1))
            s = int(g.integers(0, max(1, V - w)))
            m[r, s:s + w] = True
    m[:, 0] = True
    return m.astype(np.uint8)


@pytest.mark.parametrize("rows,V,dtype,ref,bits", [
    (12, 4104, torch.bfloat16, True, False), (6, 32000, torch.bfloat16, True, False), (3, 128256, torch.bfloat16, True, False),
    (12, 4104, torch.float32, True, False), (6, 32000, torch.float32, False, False), (3, 128256, torch.float32, True, False),
    (6, 32000, torch.bfloat16, False, False),
    (12, 4104, torch.bfloat16, True, True), (3, 128256, torch.bfloat16, True, True), (6, 32000, torch.float32, True, True)])
def test_masked_backward_values_against_oracle(oracle, rows, V, dtype, ref, bits):
    """d(logits) of rows under per-row grammar masks (whole excluded vectors: the backward kernels'
    zero-fill branch, the bf16 + reference kernel and the split f32 kernel, byte and bit masks)
    against the oracle's tape on the full [1,1,rows,V] additive −inf mask, at the reference's device
    tolerance (src/nn/tests/gpu/rl.rs:106-123: |Δ|/(1+|ref|) ≤ 1e-4 against f32, tighter against
    f64), excluded entries and unscored rows exactly zero."""
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(7 * V + rows + int(bits))
    x = g.normal(0, 3.0, (rows, V)).astype(np.float32)
    xt, xh = stored(x, dtype)
    rt = rh = None
    if ref:
        rt, rh = stored((x + g.normal(0, 0.1, (rows, V))).astype(np.float32), dtype)
    allow = _grammar_mask_np(g, rows, V)
    u = oracle.row_uniforms(V, "masked backward", rows)
    mkw = {}
    if bits:
        from test_gpu_bitmask import pack_bits

        mkw["allow_bits"] = pack_bits(allow).to(dev())
    else:
        mkw["allow"] = to_dev(allow, None)
    o = oracle.sample_inverse_cdf(xh, 1.0, u, ref_logits=rh, allow=allow)
    f = ops.row_forward(xt, ref_logits=rt, tokens=to_dev(o["tokens"].astype(np.int32), None), **mkw)
    score = np.ones(rows, np.float32)
    score[1] = 0.0
    glp, gkl, gen = (g.uniform(-1, 1, rows).astype(np.float32) * score for _ in range(3))
    d = ops.row_backward(xt, f, ref_logits=rt, g_logp=to_dev(glp, None), g_kl=to_dev(gkl, None) if ref else None, g_ent=to_dev(gen, None), **mkw).cpu().numpy().astype(np.float64)
    assert (d[allow == 0] == 0).all(), "a gradient at an excluded token"
    assert (d[1] == 0).all(), "a gradient on an unscored row"
    vm = np.where(allow != 0, 0.0, -INF)
    shape = (1, 1, rows, V)
    for dt, tol in ((oracle.F64, 2e-6), (oracle.F32, 1e-4)):
        _, want = oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, shape, dtype=dt, logits=xh, tokens=o["tokens"], vocab_mask=vm, upstream=glp)
        _, g3 = oracle.rl_eval(oracle.OP_ENTROPY, shape, dtype=dt, logits=xh, vocab_mask=vm, upstream=gen)
        want = want + g3
        if ref:
            _, g2 = oracle.rl_eval(oracle.OP_REFERENCE_KL, shape, dtype=dt, logits=xh, ref_logits=rh, vocab_mask=vm, upstream=gkl)
            want = want + g2
        err = np.abs(d.ravel() - want) / (1.0 + np.abs(want))
        assert np.nanmax(err) <= tol, f"d(logits) vs oracle dtype {dt}: {np.nanmax(err):.3e}"
        assert not np.isnan(d).any()


@pytest.mark.parametrize("rows,V", [(4, 64), (4, 4096), (3000, 4096)])
def test_kl_when_the_reference_excludes_a_token_the_policy_keeps(oracle, rows, V):
    """categorical_kl with a token excluded on one side only (src/nn/rl.rs:322-325): excluded by the
    policy → contributes 0; excluded by the reference alone → KL +inf while the policy's
    probability is positive, NaN (0·inf) once it has underflowed, exactly as Cpu(Reference) gives
    on the same inputs. Between the two underflow points (the reference's exp at −103.97, this
    library's flush-to-zero exponential at −87.34) both are non-finite: +inf there, NaN here."""
    from noetic_tensor_b200 import ops

    z = np.full((rows, V), -1.0, np.float32)
    z[:, 0] = 0.0
    zr = z.copy()
    zr[:, 5] = -INF
    shape = (1, 1, 4, V)
    for value, same_as_reference in ((-200.0, True), (-1.0, True), (-INF, True), (-95.0, False)):
        za = z.copy()
        za[:, 5] = value
        want = oracle.rl_eval(oracle.OP_KL, shape, dtype=oracle.F32, logits=za[:4], ref_logits=zr[:4])
        for dtype in (torch.float32, torch.bfloat16):
            got = ops.row_forward(to_dev(za, dtype), ref_logits=to_dev(zr, dtype)).kl.cpu().numpy()
            assert (got == got[0]).all() or np.isnan(got).all()
            if same_as_reference:
                assert np.array_equal(np.isnan(got[:4]), np.isnan(want)) and np.array_equal(np.isinf(got[:4]), np.isinf(want)), (value, got[:4], want)
                if np.isfinite(want).all():
                    assert_close(got[:4], want, "kl")
            else:
                assert np.isinf(want).all() and not np.isfinite(got).any()
    # the backward of a row whose KL is NaN is NaN throughout; the row beside it is untouched
    za = z.copy()
    za[0, 5] = -200.0
    zr2 = z.copy()
    zr2[0, 5] = -INF
    f = ops.row_forward(to_dev(za, None), ref_logits=to_dev(zr2, None))
    d = ops.row_backward(to_dev(za, None), f, ref_logits=to_dev(zr2, None), g_kl=to_dev(np.ones(rows, np.float32), None)).cpu().numpy()
    assert np.isnan(d[0]).sum() >= V - 2 and np.isfinite(d[1:]).all()
