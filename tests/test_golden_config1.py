"""The committed fixture tests/golden/config1_ppo.json (the benchmark's CPU-runnable toy: logits
[4, 2, 8, 16] f32, byte mask, one uniform per row, PPO clip 0.2): the CPU oracle must regenerate
it exactly, and the CUDA path must match it — tokens equal, values and gradients within 1e-5
relative or 1e-6 absolute."""
import importlib.util
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "config1_ppo.json")


def load():
    with open(FIXTURE) as fh:
        doc = json.load(fh)
    S, B, T, V = doc["shape"]
    a = {k: np.asarray(v) for k, v in doc["inputs"].items()}
    r = {k: np.asarray(v) for k, v in doc["results"].items()}
    return (S, B, T, V), a, r


def test_oracle_regenerates_the_fixture(oracle):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    shape, a, r = load()
    assert shape == (mg.S, mg.B, mg.T, mg.V)
    d = mg.inputs(oracle)
    for k, v in d.items():
        assert np.array_equal(np.asarray(v, dtype=np.float64).ravel(), a[k].astype(np.float64)), f"input {k}"
    out = mg.results(oracle, d)
    for k, v in out.items():
        assert np.array_equal(np.asarray(v, dtype=np.float64).ravel(), r[k].astype(np.float64)), f"result {k}"


def test_fixture_is_consistent():
    """What can be said without any implementation: tokens are allowed ones, probabilities sum to
    one, the gradient of a scored row sums to ~0 and an unscored row's is exactly zero."""
    (S, B, T, V), a, r = load()
    rows = S * B * T
    allow = a["allow"].reshape(rows, V)
    tok = r["tokens"].astype(np.int64)
    assert allow[np.arange(rows), tok].all() and (allow[:, 0] == 1).all()
    z = np.where(allow != 0, a["logits"].reshape(rows, V), -np.inf)
    lse = np.log(np.exp(z - z.max(axis=1, keepdims=True)).sum(axis=1)) + z.max(axis=1)
    assert np.allclose(r["logp"], z[np.arange(rows), tok] - lse, rtol=0, atol=2e-6)
    p = np.exp(z - lse[:, None])
    assert np.allclose(r["entropy"], -(p * np.where(p > 0, np.log(np.where(p > 0, p, 1)), 0)).sum(axis=1), atol=5e-6)
    g = r["d_logits"].reshape(rows, V)
    assert (g[a["score"] == 0] == 0).all() and np.abs(g.sum(axis=1)).max() < 1e-6
    assert (g[allow == 0] == 0).all()


def _close(got, want, what):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    ok = (np.abs(got - want) <= 1e-6) | (np.abs(got - want) <= 1e-5 * np.abs(want))
    assert ok.all(), f"{what}: worst |Δ| {np.abs(got - want).max():.3e}"


@pytest.mark.gpu
def test_cuda_path_matches_the_fixture():
    import torch

    from noetic_tensor_b200 import ops, rl

    (S, B, T, V), a, r = load()
    dev = torch.device("cuda:0")
    rows = S * B * T
    f32 = lambda v, *shape: torch.from_numpy(np.asarray(v, np.float32)).to(dev).reshape(*shape).contiguous()
    x = f32(a["logits"], S, B, T, V)
    ref = f32(a["ref"], S, B, T, V)
    allow = torch.from_numpy(a["allow"].astype(np.uint8)).to(dev).reshape(S, B, T, V)
    f = ops.row_forward(x.reshape(rows, V), ref_logits=ref.reshape(rows, V), allow=allow.reshape(rows, V), uniforms=f32(a["uniforms"], rows))
    assert (f.status == 0).all()
    assert np.array_equal(f.tokens.cpu().numpy().astype(np.int64), r["tokens"].astype(np.int64)), "no row of the fixture is a CDF boundary row"
    _close(f.logp.cpu().numpy(), r["logp"], "logp")
    _close(f.ref_logp.cpu().numpy(), r["ref_logp_f64"], "ref_logp")
    _close(f.kl.cpu().numpy(), r["kl"], "kl")
    _close(f.entropy.cpu().numpy(), r["entropy"], "entropy")
    adv = f32(np.repeat(a["adv"], T), S, B, T)
    loss = rl.clipped_policy_loss(rl.Tempered(x, 1.0, allow), f.tokens.reshape(S, B, T), f32(r["old_logp"], S, B, T), adv, f32(a["score"], S, B, T),
                                  rl.Clip.symmetric(0.2), rl.TOKEN_MEAN)
    _close(loss.value.cpu().numpy(), r["loss"], "clipped policy loss per seed")
    g = loss.backward().cpu().numpy().reshape(rows, V)
    _close(g, r["d_logits"], "d(logits)")
    assert (g[a["score"] == 0] == 0).all() and (g[a["allow"].reshape(rows, V) == 0] == 0).all()
