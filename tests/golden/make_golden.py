"""Writes tests/golden/config1_ppo.json: the CPU-runnable toy configuration of the benchmark
(logits [S=4, B=2, T=8, V=16] f32) with its inputs and the CPU oracle's results.

TEST INFRASTRUCTURE. The Rust reference cannot be built where this was written, so the values
come from the C++ restatement of `Cpu(Reference)` in oracle/ (f32 engine) and from its f64
evaluation of the inverse-CDF sampler; the fixture pins that restatement and the CUDA path to
each other and guards both against drift. Run from the repository root:

    python tests/golden/make_golden.py

Inputs, all from ChaCha20 streams of `rng::derive(seed, label)` (src/rng.rs:10-17):
  logits ~ N(0,1) seed 1; byte mask keep-probability 0.75 with token 0 always allowed; one
  uniform per row from seed 2; reference logits = logits + N(0, 0.1); old log-probs = new +
  N(0, 0.02); rewards Bernoulli(0.5) in groups of 2 -> group-relative advantages (mean only);
  PPO clip 0.2, token-mean; scoring mask with one sequence's tail padded out.
Results: tokens, log-probs, reference log-probs, exact KL and entropy per row, the clipped policy
loss per seed, and d(loss_0 + loss_1 + ...)/d(logits).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

S, B, T, V = 4, 2, 8, 16
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config1_ppo.json")


def unit_floats(orc, seed, label, n):
    """n doubles in (0, 1) from a derived ChaCha20 stream: (w + 0.5) / 2^32."""
    w = orc.chacha20_words(orc.derive_seed(seed, label), n)
    return (w.astype(np.float64) + 0.5) / 4294967296.0


def normals(orc, seed, label, n):
    """Box-Muller on pairs of the stream's uniforms."""
    u = unit_floats(orc, seed, label, 2 * n)
    return np.sqrt(-2.0 * np.log(u[0::2])) * np.cos(2.0 * np.pi * u[1::2])


def inputs(orc):
    rows = S * B * T
    logits = normals(orc, 1, "logits", rows * V).astype(np.float32).reshape(rows, V)
    allow = (unit_floats(orc, 1, "mask", rows * V) < 0.75).astype(np.uint8).reshape(rows, V)
    allow[:, 0] = 1
    uniforms = orc.row_uniforms(2, "uniforms", rows)
    ref = (logits.astype(np.float64) + 0.1 * normals(orc, 1, "reference", rows * V).reshape(rows, V)).astype(np.float32)
    rewards = (unit_floats(orc, 1, "rewards", S * B) < 0.5).astype(np.float64)
    adv = orc.group_advantages(rewards, 2, norm="mean")  # [S*B], one per sequence
    score = np.ones((S, B, T))
    score[1, 1, 5:] = 0.0  # padding
    score[3, 0, 7:] = 0.0
    return dict(logits=logits, allow=allow, uniforms=uniforms, ref=ref, rewards=rewards, adv=adv, score=score.reshape(-1))


def results(orc, d):
    rows = S * B * T
    shape = (S, B, T, V)
    o = orc.sample_inverse_cdf(d["logits"], 1.0, d["uniforms"], ref_logits=d["ref"], allow=d["allow"])
    assert (o["status"] == 0).all()
    vm = np.where(d["allow"] != 0, 0.0, -np.inf)
    tokens = o["tokens"]
    logp = orc.rl_eval(orc.OP_TOKEN_LOG_PROBS, shape, logits=d["logits"], tokens=tokens, vocab_mask=vm)
    kl = orc.rl_eval(orc.OP_REFERENCE_KL, shape, logits=d["logits"], ref_logits=d["ref"], vocab_mask=vm, reduction=orc.NONE)
    ent = orc.rl_eval(orc.OP_ENTROPY, shape, logits=d["logits"], vocab_mask=vm, reduction=orc.NONE)
    old = logp + 0.02 * normals(orc, 1, "old", rows)
    old = old.astype(np.float32).astype(np.float64)
    w = np.repeat(d["adv"], T).reshape(S, B, T)
    loss, grad = orc.rl_eval(orc.OP_PPO, shape, logits=d["logits"], tokens=tokens, old_logp=old, weights=w, mask=d["score"], vocab_mask=vm,
                             clip=orc.Clip.symmetric(0.2), reduction=orc.TOKEN_MEAN, upstream=np.ones(S))
    return dict(tokens=tokens, boundary=o["boundary"], logp=logp, ref_logp_f64=o["ref_logp"], kl=kl, entropy=ent, old_logp=old, loss=loss, d_logits=grad.reshape(rows, V))


def main():
    import oracle as orc

    orc.build()
    orc.set_backend(False, 1)
    d = inputs(orc)
    r = results(orc, d)
    doc = {"shape": [S, B, T, V], "clip": 0.2, "reduction": "token_mean",
           "inputs": {k: (v.astype(np.float64) if v.dtype.kind == "f" else v).ravel().tolist() for k, v in d.items()},
           "results": {k: (v.astype(np.float64) if v.dtype.kind == "f" else v).ravel().tolist() for k, v in r.items()}}
    with open(OUT, "w") as fh:
        json.dump(doc, fh, separators=(",", ":"))
        fh.write("\n")
    print(OUT, os.path.getsize(OUT), "bytes;", int(r["boundary"].sum()), "boundary rows")


if __name__ == "__main__":
    main()
