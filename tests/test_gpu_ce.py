"""GPU parity of the cross-entropy family (nn::loss over the fused row kernels, through the C
ABI) against the CPU oracle's restatement of src/nn/loss.rs: values within 1e-5 and gradients
within 1e-4 by |Δ|/(1+|ref|) of the f32 reference engine (the reference's own device gates,
src/nn/tests/gpu/rl.rs:16-19) and within 1e-5 rel / 1e-6 abs of the f64 engine; bitwise equal
run to run."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def rel(got, want):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape
    e = np.abs(got - want) / (1.0 + np.abs(want))
    return float(np.where(got == want, 0.0, e).max()) if got.size else 0.0


def close(got, want, what, rel_=1e-5, abs_=1e-6):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    err = np.abs(got - want)
    ok = (got == want) | (err <= abs_) | (err <= rel_ * np.abs(want))
    assert ok.all(), f"{what}: worst |Δ| {err[~ok].max():.3e}"


def stored(x, dtype):
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dev()).to(dtype)
    host = t.view(torch.int16).cpu().numpy().view(np.uint16) if dtype == torch.bfloat16 else t.cpu().numpy()
    return t, host


CASES = [((3, 2, 4, 5), torch.float32), ((2, 2, 3, 5), torch.float32), ((2, 3, 8, 37), torch.bfloat16), ((2, 2, 16, 1000), torch.bfloat16),
         ((1, 2, 3, 4104), torch.float32), ((2, 1, 2, 32000), torch.bfloat16)]


@pytest.mark.parametrize("shape,dtype", CASES)
def test_cross_entropy_family_matches_the_reference_engine(oracle, shape, dtype):
    from noetic_tensor_b200 import loss

    S, B, T, V = shape
    n = S * B * T
    g = np.random.default_rng(V + n)
    x, xh = stored(g.uniform(-3, 3, shape), dtype)
    tg = g.integers(0, V, (S, B, T))
    mask = (g.uniform(0, 1, (S, B, T)) < 0.6).astype(np.float32)
    mask[-1] = 0.0  # the last seed scores nothing
    tg_ign = tg.copy()
    tg_ign.ravel()[[1, n // 2]] = -100
    tgt, tgt_ign, mt = torch.from_numpy(tg).to(dev()), torch.from_numpy(tg_ign).to(dev()), torch.from_numpy(mask).to(dev())
    up = g.uniform(0.5, 1.5, S)
    upt = torch.from_numpy(up.astype(np.float32)).to(dev())
    runs = [
        ("nll", oracle.OP_NLL, lambda: loss.nll(x, tgt), dict(tokens=tg), g.uniform(0.5, 1.5, n)),
        ("cross_entropy", oracle.OP_CE, lambda: loss.cross_entropy(x, tgt), dict(tokens=tg), up),
        ("masked_cross_entropy", oracle.OP_MASKED_CE, lambda: loss.masked_cross_entropy(x, tgt, mt), dict(tokens=tg, mask=mask), up),
        ("ignore_index", oracle.OP_CE_WITH, lambda: loss.cross_entropy_with(x, tgt_ign, mt, loss.CeOptions(ignore_index=-100)), dict(tokens=tg_ign, mask=mask, ignore_index=-100), up),
        ("smoothing", oracle.OP_CE_WITH, lambda: loss.cross_entropy_with(x, tgt_ign, mt, loss.CeOptions(ignore_index=-100, smoothing=0.1)), dict(tokens=tg_ign, mask=mask, ignore_index=-100, smoothing=0.1), up),
        ("smoothing, unmasked", oracle.OP_CE_WITH, lambda: loss.cross_entropy_with(x, tgt, None, loss.CeOptions(smoothing=0.3)), dict(tokens=tg, smoothing=0.3), up),
    ]
    for name, op, run, kw, u in runs:
        l = run()
        ut = torch.from_numpy(np.asarray(u, np.float32)).to(dev()).reshape(l.value.shape)
        d = l.backward(ut)
        u32 = np.asarray(u, np.float32).astype(np.float64)
        v32, g32 = oracle.rl_eval(op, shape, dtype=oracle.F32, logits=xh, upstream=u32, **kw)
        v64, g64 = oracle.rl_eval(op, shape, dtype=oracle.F64, logits=xh, upstream=u32, **kw)
        got_v, got_g = l.value.cpu().numpy(), d.cpu().numpy()
        assert rel(got_v, v32) <= 1e-5 and rel(got_g, g32) <= 1e-4, (name, rel(got_v, v32), rel(got_g, g32))
        close(got_v, v64, name + " value")
        close(got_g, g64, name + " gradient", rel_=1e-5, abs_=1e-6)
        if "mask" in kw:
            assert got_v.ravel()[-1] == 0.0, "a seed with no scored position has loss 0"
            dz = got_g.reshape(n, V)
            assert (dz[mask.ravel() == 0] == 0).all(), "an unscored position has a gradient"
        l2 = run()
        assert torch.equal(l2.value.view(torch.int32), l.value.view(torch.int32)) and torch.equal(l2.backward(ut).view(torch.int32), d.view(torch.int32)), name
    # default options are the plain losses, to the bit (src/nn/tests/components.rs:566-569)
    a = loss.cross_entropy_with(x, tgt, mt, loss.CeOptions()).value
    b = loss.masked_cross_entropy(x, tgt, mt).value
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    # ignore_index = masked CE with those positions masked out and class 0 as target, to the bit (:559-565)
    m2, tg2 = mask.copy(), tg_ign.copy()
    m2[tg_ign == -100] = 0.0
    tg2[tg_ign == -100] = 0
    a = loss.cross_entropy_with(x, tgt_ign, mt, loss.CeOptions(ignore_index=-100)).value
    b = loss.masked_cross_entropy(x, torch.from_numpy(tg2).to(dev()), torch.from_numpy(m2).to(dev())).value
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("shape,dtype", [((2, 2, 3, 5), torch.float32), ((2, 3, 4, 1000), torch.bfloat16), ((1, 1, 6, 4104), torch.float32)])
def test_kl_div_and_both_gradients(oracle, shape, dtype):
    from noetic_tensor_b200 import loss

    S, B, T, V = shape
    g = np.random.default_rng(V)
    q, qh = stored(g.uniform(-2, 2, shape), dtype)
    p, ph = stored(g.uniform(-2, 2, shape), dtype)
    up = g.uniform(0.5, 1.5, S).astype(np.float32)
    l = loss.kl_div(q, p)
    dq, dp = l.backward(torch.from_numpy(up).to(dev()), wrt_target=True)
    v32, gq32, gp32 = oracle.rl_eval(oracle.OP_KL_DIV, shape, dtype=oracle.F32, logits=qh, ref_logits=ph, upstream=up.astype(np.float64), grad_ref=True)
    v64, gq64, gp64 = oracle.rl_eval(oracle.OP_KL_DIV, shape, dtype=oracle.F64, logits=qh, ref_logits=ph, upstream=up.astype(np.float64), grad_ref=True)
    assert rel(l.value.cpu().numpy(), v32) <= 1e-5 and rel(dq.cpu().numpy(), gq32) <= 1e-4 and rel(dp.cpu().numpy(), gp32) <= 1e-4
    close(l.value.cpu().numpy(), v64, "kl_div")
    close(dq.cpu().numpy(), gq64, "d kl_div / d pred")
    close(dp.cpu().numpy(), gp64, "d kl_div / d target")
    assert (l.value >= 0).all()
    only_q = l.backward(torch.from_numpy(up).to(dev()))
    assert torch.equal(only_q.view(torch.int32), dq.view(torch.int32))
    same = loss.kl_div(q, q).value
    assert (same.abs() < 1e-6).all()


def test_errors_follow_the_reference():
    from noetic_tensor_b200 import loss

    x = torch.zeros(1, 1, 2, 4, device=dev())
    with pytest.raises(IndexError, match="one_hot: 4 is outside 0..4"):
        loss.cross_entropy(x, torch.tensor([[[0, 4]]], device=dev()))
    with pytest.raises(IndexError, match="one_hot: -100"):
        loss.cross_entropy(x, torch.tensor([[[0, -100]]], device=dev()))
    with pytest.raises(ValueError, match="label smoothing 1.5 outside"):
        loss.cross_entropy_with(x, torch.tensor([[[0, 1]]], device=dev()), None, loss.CeOptions(smoothing=1.5))
    # a target the logits exclude at an unscored position: the mask is a product, as in the reference
    x[0, 0, 1, 2] = float("-inf")
    l = loss.masked_cross_entropy(x, torch.tensor([[[0, 2]]], device=dev()), torch.tensor([[[1.0, 0.0]]], device=dev()))
    assert torch.isnan(l.value).all()


def test_pretraining_shape_full_vocabulary(oracle):
    """V = 128256 bf16, 2048 positions per seed: properties at a size the oracle cannot finish,
    plus the oracle on a sample of rows."""
    from noetic_tensor_b200 import loss, ops, synth

    gen = torch.Generator(device=dev())
    gen.manual_seed(9)
    S, B, T, V = 2, 2, 1024, 128256
    rows = S * B * T
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev()).reshape(S, B, T, V)
    tg = torch.randint(0, V, (S, B, T), generator=gen, device=dev())
    mask = (torch.rand(S, B, T, generator=gen, device=dev()) < 0.9).float()
    eps = 0.1
    l = loss.cross_entropy_with(x, tg, mask, loss.CeOptions(smoothing=eps))
    d = l.backward().reshape(rows, V)
    assert torch.isfinite(l.value).all() and (l.value > 0).all()
    count = mask.reshape(S, -1).sum(1).clamp_min(1.0).repeat_interleave(B * T)
    assert d.sum(dim=1).abs().max().item() < 1e-6, "rows of a softmax-minus-distribution gradient sum to 0"
    assert (d[mask.reshape(-1) == 0] == 0).all()
    # the target's entry: keep/count · (π_t − (1 − ε) − ε/V)
    f = ops.row_forward(x.reshape(rows, V), tokens=tg.reshape(-1).int(), want_entropy=False)
    want = mask.reshape(-1) / count * (torch.exp(f.logp) - (1 - eps) - eps / V)
    got = d[torch.arange(rows, device=dev()), tg.reshape(-1)]
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-9)
    # oracle on 24 rows: nll and the uniform term through an unmasked, unreduced evaluation
    idx = torch.from_numpy(np.random.default_rng(1).choice(rows, 24, replace=False)).to(dev())
    xs = x.reshape(rows, V)[idx].contiguous()
    sub = loss.cross_entropy_with(xs.reshape(24, 1, 1, V), tg.reshape(-1)[idx].reshape(24, 1, 1), None, loss.CeOptions(smoothing=eps))
    xh = xs.view(torch.int16).cpu().numpy().view(np.uint16)
    v64 = oracle.rl_eval(oracle.OP_CE_WITH, (24, 1, 1, V), dtype=oracle.F64, logits=xh, tokens=tg.reshape(-1)[idx].cpu().numpy(), smoothing=eps)
    close(sub.value.cpu().numpy(), v64, "smoothed CE at V = 128256")
