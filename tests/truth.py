"""Host f64 formulas of the reference's own tests (src/nn/tests/rl.rs), in numpy.

These are an implementation independent of the C++ oracle: log_softmax_host (:19-27),
reduce_host (:30-54), ppo_host_full (:656-672), kl_host / entropy_host (:336-343), k_host (:427-434).
"""
import numpy as np


def log_softmax_host(x, v):
    x = np.asarray(x, dtype=np.float64).reshape(-1, v)
    m = x.max(axis=1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = np.log(np.exp(x - m).sum(axis=1, keepdims=True)) + m
        return x - lse


def reduce_host(per, mask, shape, r):
    s, b, t = shape
    per = np.asarray(per, dtype=np.float64).reshape(s, b, t)
    mask = np.asarray(mask, dtype=np.float64).reshape(s, b, t)
    seq_v, seq_n = per.sum(axis=2), mask.sum(axis=2)
    if r == 0:
        return per.ravel()
    if r == 1:
        return seq_v.sum(axis=1)
    if r == 2:
        return seq_v.sum(axis=1) / np.maximum(seq_n.sum(axis=1), 1.0)
    if r == 3:
        return (seq_v / np.maximum(seq_n, 1.0)).ravel()
    if r == 4:
        ps = np.where(seq_n > 0, seq_v / np.maximum(seq_n, 1.0), 0.0)
        return ps.sum(axis=1) / np.maximum((seq_n > 0).sum(axis=1), 1.0)
    raise ValueError(r)


def ppo_host_full(lp, old, adv, mask, low, high, dual=None, log_ratio_clamp=None):
    lp, old, adv, mask = (np.asarray(a, dtype=np.float64).ravel() for a in (lp, old, adv, mask))
    d = lp - old
    if log_ratio_clamp is not None:
        d = np.clip(d, -log_ratio_clamp, log_ratio_clamp)
    with np.errstate(over="ignore", invalid="ignore"):
        r = np.exp(d)
        l = np.maximum(-(r * adv), -(np.clip(r, 1.0 - low, 1.0 + high) * adv))
        if dual is not None:
            l = np.where(adv < 0.0, np.minimum(l, -dual * adv), l)
    return np.where(mask == 0.0, 0.0, l)


def kl_host(p, q, v):
    lp, lq = log_softmax_host(p, v), log_softmax_host(q, v)
    with np.errstate(invalid="ignore", over="ignore"):
        term = np.where(lp == -np.inf, 0.0, np.exp(lp) * (lp - lq))
    return term.sum(axis=1)


def entropy_host(x, v):
    lp = log_softmax_host(x, v)
    with np.errstate(invalid="ignore"):
        term = np.where(lp == -np.inf, 0.0, np.exp(lp) * lp)
    return -term.sum(axis=1)


def k_host(lp, lr, e):
    d = np.asarray(lr, dtype=np.float64) - np.asarray(lp, dtype=np.float64)
    with np.errstate(over="ignore"):
        return {1: -d, 2: d * d / 2.0, 3: np.exp(d) - d - 1.0}[e]


class Case:
    """The reference tests' batch (src/nn/tests/rl.rs:58-76): S 2, B 3, T 4, V 5; sequence 2 of
    seed 1 entirely masked, sequence 0 of seed 0 with one scored token, the rest random. The
    reference draws it from ChaCha8; here numpy's generator supplies the same shapes and ranges."""

    def __init__(self, seed, lo, hi, s=2, b=3, t=4, v=5):
        g = np.random.default_rng(seed)
        self.sh = (s, b, t)
        self.v = v
        n = s * b * t
        self.n = n
        self.logits = g.uniform(lo, hi, n * v)
        self.tokens = g.integers(0, v, n)
        mask = (g.uniform(0, 1, n) < 0.7).astype(np.float64)
        mask[0:t] = [0.0, 1.0, 0.0, 0.0][:t] if t == 4 else 0.0
        z = (b + 2) * t
        mask[z:z + t] = 0.0
        self.mask = mask

    @property
    def lshape(self):
        return (*self.sh, self.v)

    def logp_host(self):
        lp = log_softmax_host(self.logits, self.v)
        return lp[np.arange(self.n), self.tokens]


# ---- the operand order of the library's TokenReduction kernels, for bit comparisons -------------
# Step 1 (one warp per sequence): lane l adds the elements l, l + 32, ... in order in f32, then the
# 32 lane sums meet in a butterfly (xor 16, 8, 4, 2, 1). Step 2: a seed's pairs folded in sequence
# order in f64. tests/test_gpu_losses.py holds nrl_reduce_tokens to these bits on the GPU, and
# tests/test_shard_gloo.py runs the multi-rank plumbing over them on the CPU.

def warp_seq_pairs(per, mask):
    per = np.asarray(per, dtype=np.float32)
    n_seq, T = per.shape
    mask = np.ones_like(per) if mask is None else np.asarray(mask, dtype=np.float32)
    out = np.zeros((n_seq, 2), dtype=np.float32)
    for k, x in enumerate((per, mask)):
        pad = (-T) % 32
        xp = np.concatenate([x, np.zeros((n_seq, pad), np.float32)], axis=1).reshape(n_seq, -1, 32)
        lanes = np.zeros((n_seq, 32), dtype=np.float32)
        for j in range(xp.shape[1]):
            # a lane past the end of the sequence adds nothing (the kernel's loop simply ends)
            live = (j * 32 + np.arange(32)) < T
            lanes = np.where(live, (lanes + xp[:, j, :]).astype(np.float32), lanes)
        for s in (16, 8, 4, 2, 1):
            lanes = (lanes + lanes[:, np.arange(32) ^ s]).astype(np.float32)
        out[:, k] = lanes[:, 0]
    return out


def fold_pairs(pairs, S, B, reduction):
    pairs = np.asarray(pairs, dtype=np.float32).reshape(S, B, 2)
    v, c = pairs[..., 0], pairs[..., 1]
    ps = (v / np.maximum(c, np.float32(1.0))).astype(np.float32)
    if reduction == 3:
        return ps
    out = np.zeros(S, dtype=np.float32)
    for s in range(S):
        tot = count = seq_tot = nonempty = 0.0
        for b in range(B):
            tot += float(v[s, b])
            count += float(c[s, b])
            seq_tot += float(ps[s, b])
            nonempty += float(min(c[s, b], np.float32(1.0)))
        if reduction == 1:
            out[s] = np.float32(tot)
        elif reduction == 2:
            out[s] = np.float32(tot) / max(np.float32(count), np.float32(1.0))
        else:
            out[s] = np.float32(seq_tot) / max(np.float32(nonempty), np.float32(1.0))
    return out


def bwd_pairs(reduction, S, B, T, seq_begin, n_seq, pairs, mask, g_out):
    pairs = np.asarray(pairs, dtype=np.float32).reshape(S, B, 2)
    g_out = np.asarray(g_out, dtype=np.float32)
    d = np.zeros((n_seq, T), dtype=np.float32)
    for q in range(n_seq):
        seq = seq_begin + q
        s = seq // B
        cnt = float(pairs[s, :, 1].astype(np.float64).sum())
        non = float(np.minimum(pairs[s, :, 1], np.float32(1.0)).astype(np.float64).sum())
        seq_scale = max(pairs[s, seq % B, 1], np.float32(1.0))
        if reduction == 3:
            g = g_out.reshape(-1)[seq] / seq_scale
        elif reduction == 4:
            g = (g_out[s] / max(np.float32(non), np.float32(1.0))) / seq_scale
        elif reduction == 2:
            g = g_out[s] / max(np.float32(cnt), np.float32(1.0))
        else:
            g = g_out[s]
        d[q] = np.float32(g)
    if mask is not None:
        d = np.where(np.asarray(mask) != 0, d, np.float32(0.0))
    return d
