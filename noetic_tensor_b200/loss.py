"""The cross-entropy family of noetic-tensor's `nn::loss` (src/nn/loss.rs:10-79, 175-183) on the
fused row kernels: same names, argument meanings, per-seed results `[S]` and error behaviour.

Where the reference runs log_softmax, builds a dense one-hot `[S, N, V]`, multiplies and sums
(three `[rows, V]` f32 intermediates plus the saved log-softmax), this reads the logits once
forward (twice with label smoothing) and once backward. Each function returns an `rl.Loss`:
`.value` and `.backward(upstream)` → d(logits) `[S, B, T, V]` f32 (kl_div: a pair).
"""
import torch

from . import capi, ops
from .rl import Loss


class CeOptions:
    """`CeOptions` (src/nn/loss.rs:36-43)."""

    def __init__(self, ignore_index=None, smoothing=0.0):
        self.ignore_index, self.smoothing = ignore_index, smoothing

    def is_default(self):
        return self.ignore_index is None and self.smoothing == 0.0


def _rows(logits):
    if logits.dim() != 4:
        raise ValueError("logits [S, B, T, V]")
    S, B, T, V = logits.shape
    return S, B * T, V, logits.reshape(S * B * T, V)


def _targets(targets, S, N, V, ignore_index=None):
    """Targets as device I32 rows and the not-ignored weights; ignored targets read class 0
    (src/nn/loss.rs:60-65). An out-of-range target is the reference's one_hot error."""
    t = targets.reshape(-1).to(torch.int64)
    if t.numel() != S * N:
        raise ValueError("targets [S, B, T]")
    keep = None
    if ignore_index is not None:
        ignored = t == ignore_index
        keep = (~ignored).to(torch.float32)
        t = torch.where(ignored, torch.zeros_like(t), t)
    bad = (t < 0) | (t >= V)
    if bad.any():
        raise IndexError(f"one_hot: {int(t[bad][0])} is outside 0..{V}")
    return t.to(torch.int32).contiguous(), keep


def _ce(logits, targets, keep, smoothing, reduce):
    S, N, V, flat = _rows(logits)
    tok, not_ignored = targets
    if keep is not None and not_ignored is not None:
        keep = keep * not_ignored
    elif not_ignored is not None:
        keep = not_ignored
    fwd = ops.row_forward(flat, tokens=tok, want_entropy=False)
    zsum = ops.row_sum(flat) if smoothing > 0.0 else None
    per, _, _ = ops.ce_tokens(V, fwd.logp, smoothing=smoothing, rowstats=fwd.rowstats, logit_sum=zsum, keep=keep)
    per3 = per.reshape(S, 1, N)
    keep3 = None if keep is None else keep.reshape(S, 1, N)
    value = ops.reduce_tokens(per3, keep3, capi.REDUCE_TOKEN_MEAN) if reduce else per.reshape(S, N)

    def backward(up):
        if reduce:
            d_per = ops.reduce_tokens_backward((S, 1, N), keep3, capi.REDUCE_TOKEN_MEAN, up.reshape(S))
        else:
            d_per = up
        _, g_lp, g_un = ops.ce_tokens(V, fwd.logp, smoothing=smoothing, rowstats=fwd.rowstats, logit_sum=zsum, keep=keep,
                                      upstream=d_per.reshape(-1).contiguous(), want_loss=False)
        return ops.row_backward(flat, fwd, g_logp=g_lp, g_uniform=g_un).reshape(logits.shape)

    return Loss(value, backward)


def nll(logits, targets):
    """Per-token negative log-likelihood `[S, B·T]` (src/nn/loss.rs:10-16)."""
    S, N, V, _ = _rows(logits)
    return _ce(logits, _targets(targets, S, N, V), None, 0.0, reduce=False)


def cross_entropy(logits, targets):
    """Per-seed mean cross-entropy over every position, `[S]` (src/nn/loss.rs:19-22)."""
    S, N, V, _ = _rows(logits)
    return _ce(logits, _targets(targets, S, N, V), None, 0.0, reduce=True)


def masked_cross_entropy(logits, targets, mask):
    """`sum(nll · mask) / max(count, 1)` per seed (src/nn/loss.rs:27-34)."""
    S, N, V, _ = _rows(logits)
    keep = mask.reshape(S * N).to(torch.float32).contiguous()
    return _ce(logits, _targets(targets, S, N, V), keep, 0.0, reduce=True)


def cross_entropy_with(logits, targets, mask=None, opts=None):
    """Mask, `ignore_index` and label smoothing (src/nn/loss.rs:48-79)."""
    opts = opts or CeOptions()
    if opts.is_default():
        return masked_cross_entropy(logits, targets, mask) if mask is not None else cross_entropy(logits, targets)
    if not 0.0 <= opts.smoothing <= 1.0:
        raise ValueError(f"label smoothing {opts.smoothing} outside [0, 1]")
    S, N, V, _ = _rows(logits)
    keep = None if mask is None else mask.reshape(S * N).to(torch.float32).contiguous()
    return _ce(logits, _targets(targets, S, N, V, opts.ignore_index), keep, float(opts.smoothing), reduce=True)


def kl_div(pred_logits, target_logits):
    """Per-seed mean over positions of KL(softmax(target) ‖ softmax(pred)) (src/nn/loss.rs:175-183).
    `.backward(up, wrt_target=False)` returns d(pred_logits), and with `wrt_target=True` the pair
    (d(pred_logits), d(target_logits))."""
    if pred_logits.shape != target_logits.shape:
        raise ValueError("kl_div: shapes differ")
    S = pred_logits.shape[0]
    V = pred_logits.shape[-1]
    q = pred_logits.reshape(-1, V)
    p = target_logits.reshape(-1, V)
    N = q.shape[0] // S
    fwd = ops.row_forward(p, ref_logits=q, want_logp=False, want_entropy=False)  # policy side = target
    value = ops.reduce_tokens(fwd.kl.reshape(S, 1, N), None, capi.REDUCE_TOKEN_MEAN)

    def backward(up, wrt_target=False):
        g = ops.reduce_tokens_backward((S, 1, N), None, capi.REDUCE_TOKEN_MEAN, up.reshape(S)).reshape(-1).contiguous()
        d_p, d_q = ops.row_backward(p, fwd, ref_logits=q, g_kl=g, d_ref=True, want_d_logits=wrt_target)
        d_q = d_q.reshape(pred_logits.shape)
        return (d_q, d_p.reshape(pred_logits.shape)) if wrt_target else d_q

    loss = Loss(value, None)
    loss.backward = lambda upstream=None, wrt_target=False: backward((torch.ones_like(value) if upstream is None else upstream).to(torch.float32).contiguous(), wrt_target)
    return loss
