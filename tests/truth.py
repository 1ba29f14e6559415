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
