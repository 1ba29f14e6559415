"""`nn::rl` over the fused kernels: the reference's function names and argument meanings
(src/nn/rl.rs), for logits that live on a CUDA device.

Each loss returns a `Loss`: `.value` is the reduced tensor the reference function returns and
`.backward(upstream)` gives d(logits) [S,B,T,V] f32 for sum(value · upstream), what the tape's
`(value * upstream).sum().backward()` yields in the reference. Where the reference builds ~40
tape nodes per PPO step, this path has one forward and one backward pass over the logits.

Masks: `mask` is the scoring mask [S,B,T] of 0/1 floats (src/nn/rl.rs:9-14); `vocab_mask` is
either a float additive mask broadcastable as [1,V] or [rows,V] (the reference's form,
src/nn/rl.rs:471-486) or a uint8/bool allow-mask of the same shapes.
"""
import os

import torch

from . import capi, ops

NONE, SUM, TOKEN_MEAN, PER_SEQUENCE, SEQUENCE_MEAN = range(5)
K1, K2, K3 = capi.LOSS_K1, capi.LOSS_K2, capi.LOSS_K3
LOG_RATIO_CLAMP = 20.0  # src/nn/rl.rs:146
KL_DELTA_CLAMP = 20.0  # src/nn/rl.rs:150


# The reference's losses check their scored log-probabilities in debug builds only
# (`debug_check`, src/nn/rl.rs:213-221: a host read). Here the switch is this flag, set from the
# environment variable NOETIC_RL_DEBUG (any value but "" and "0") when the module is imported.
DEBUG_CHECKS = os.environ.get("NOETIC_RL_DEBUG", "0") not in ("", "0")


def check_scored_finite(what, logp, mask=None):
    """`check_scored_finite` (src/nn/rl.rs:204-211): None, or the error text naming the first scored
    position whose log-probability is not finite."""
    return ops.check_scored_finite(what, logp.contiguous(), None if mask is None else mask.contiguous())


def debug_check(what, logp, mask=None):
    """`debug_check` (src/nn/rl.rs:213-221): raises the check's message when DEBUG_CHECKS is on."""
    if DEBUG_CHECKS:
        e = check_scored_finite(what, logp, mask)
        if e is not None:
            raise RuntimeError(e)


class Clip:
    """`Clip` (src/nn/rl.rs:160-198)."""

    def __init__(self, low, high, dual=None, log_ratio_clamp=LOG_RATIO_CLAMP):
        self.low, self.high, self.dual, self.log_ratio_clamp = low, high, dual, log_ratio_clamp

    @staticmethod
    def symmetric(eps):
        return Clip(eps, eps)

    def with_dual(self, c):
        return Clip(self.low, self.high, c, self.log_ratio_clamp)

    def with_log_ratio_clamp(self, b):
        return Clip(self.low, self.high, self.dual, b)


class Tempered:
    """`tempered_logits(logits, temperature, mask)` (src/nn/rl.rs:475-486) without materialising
    it: the kernels apply the temperature and the mask as they stream the row."""

    def __init__(self, logits, temperature=1.0, vocab_mask=None):
        if not (temperature > 0.0):
            raise ValueError(f"tempered_logits: temperature {temperature} (must be positive)")
        self.logits = logits
        self.shape = tuple(logits.shape)
        self.V = logits.shape[-1]
        self.flat = logits.reshape(-1, self.V)
        self.temperature = float(temperature)
        self.allow = self.add = None
        if vocab_mask is not None:
            if vocab_mask.shape[-1] != self.V:
                raise ValueError("tempered_logits: mask does not broadcast to the logits")
            m = vocab_mask.reshape(-1, self.V)
            if m.dtype in (torch.uint8, torch.bool):
                self.allow = m.contiguous()
            else:
                self.add = m.to(torch.float32).contiguous()

    def kw(self):
        return dict(allow=self.allow, add_mask=self.add, temperature=self.temperature)


def _tempered(x):
    return x if isinstance(x, Tempered) else Tempered(x)


class Loss:
    def __init__(self, value, backward):
        self.value = value
        self._backward = backward

    def backward(self, upstream=None):
        if upstream is None:
            upstream = torch.ones_like(self.value)
        return self._backward(upstream.to(torch.float32).contiguous())


def sample_categorical(logits, temperature=1.0, vocab_mask=None, uniforms=None):
    """Tokens [...] (int32) from softmax(logits/τ + mask): inverse CDF against `uniforms` (one per
    position); τ = 0 is the first maximum. Refuses a position with no allowed token or a NaN with
    the reference's message (src/nn/rl.rs:516-519). Returns (tokens, log-probs of the tokens)."""
    if temperature < 0:
        raise ValueError(f"sample_categorical: temperature {temperature} (must be ≥ 0)")
    z = Tempered(logits, 1.0 if temperature == 0.0 else temperature, vocab_mask)
    lead = z.shape[:-1]
    if temperature == 0.0:
        f = ops.row_forward(z.flat, greedy=True, want_entropy=False, **z.kw())
    else:
        f = ops.row_forward(z.flat, uniforms=uniforms.reshape(-1).contiguous(), want_entropy=False, **z.kw())
    ops.check_status(f.status)
    return f.tokens.reshape(lead), f.logp.reshape(lead)


class ChaChaStream:
    """The position of a `ChaCha20Rng` (src/rng.rs:10-17 derives its 32-byte seed): the seed and
    the number of 32-bit words drawn so far. `sample_categorical_reference` advances it as the
    reference's sampler advances its generator."""

    def __init__(self, seed, words=0):
        if len(seed) != 32:
            raise ValueError("seed: 32 bytes")
        self.seed, self.words = bytes(seed), int(words)


def sample_categorical_reference(logits, temperature, vocab_mask, rng):
    """`sample_categorical(logits, temperature, mask, rng)` with the reference's own noise
    (src/nn/rl.rs:510-529): Gumbel-max, one `next_u64` of `rng` per logit in row-major order, so the
    tokens are the reference's for the same generator state. Temperature 0 is the first maximum
    and draws nothing. Refuses a position with no allowed token before drawing, as the reference
    does. Returns tokens [...] (int32)."""
    if temperature < 0:
        raise ValueError(f"sample_categorical: temperature {temperature} (must be ≥ 0)")
    z = Tempered(logits, 1.0 if temperature == 0.0 else temperature, vocab_mask)
    lead = z.shape[:-1]
    if temperature == 0.0:
        f = ops.row_forward(z.flat, greedy=True, want_entropy=False, want_logp=False, **z.kw())
        ops.check_status(f.status)
        return f.tokens.reshape(lead)
    tokens, status = ops.sample_gumbel(z.flat, rng.seed, word_offset=rng.words, **z.kw())
    ops.check_status(status)
    rng.words += 2 * z.flat.shape[0] * z.V
    return tokens.reshape(lead)


class _TokenLogProbs:
    """token_log_probs (src/nn/rl.rs:134-141) and its backward to the logits."""

    def __init__(self, logits, tokens):
        self.z = _tempered(logits)
        self.lead = self.z.shape[:-1]
        self.fwd = ops.row_forward(self.z.flat, tokens=tokens.reshape(-1).to(torch.int32).contiguous(), want_entropy=False, **self.z.kw())
        self.logp = self.fwd.logp.reshape(self.lead)

    def grad_logits(self, g_logp):
        d = ops.row_backward(self.z.flat, self.fwd, g_logp=g_logp.reshape(-1).contiguous(), **self.z.kw())
        return d.reshape(self.z.shape)


def token_log_probs(logits, tokens, mask=None):
    t = _TokenLogProbs(logits, tokens)
    value = t.logp if mask is None else ops.mask_rows(t.logp, mask)

    def backward(up):
        g = up if mask is None else ops.mask_rows(up, mask)
        return t.grad_logits(g)

    return Loss(value, backward)


_CHECK_NAMES = {
    capi.LOSS_PG: ("policy_gradient_loss", None),
    capi.LOSS_PPO: ("clipped_policy_loss", "clipped_policy_loss (old log-probabilities)"),
    capi.LOSS_K1: ("kl_estimate", "kl_estimate (reference log-probabilities)"),
    capi.LOSS_K2: ("kl_estimate", "kl_estimate (reference log-probabilities)"),
    capi.LOSS_K3: ("kl_estimate", "kl_estimate (reference log-probabilities)"),
}


def _token_level(kind, logits, tokens, mask, reduction, **kw):
    t = _TokenLogProbs(logits, tokens)
    lp = t.logp.reshape(t.lead) if len(t.lead) == 3 else None
    if lp is None:
        raise ValueError("logp must be [S, B, T]")
    # the checks of src/nn/rl.rs:230, 268-269, 386-387
    what, what_other = _CHECK_NAMES[kind]
    debug_check(what, lp, mask)
    if what_other is not None:
        debug_check(what_other, kw["other"], mask)
    per, _ = ops.token_loss(kind, lp, mask=mask, want_grad=False, **kw)
    value = ops.reduce_tokens(per, mask, reduction)

    def backward(up):
        d_per = ops.reduce_tokens_backward(tuple(lp.shape), mask, reduction, up)
        _, g_logp = ops.token_loss(kind, lp, mask=mask, upstream=d_per, **kw)
        return t.grad_logits(g_logp)

    return Loss(value, backward)


def policy_gradient_loss(logits, tokens, weights, mask=None, reduction=TOKEN_MEAN):
    """policy_gradient_loss(token_log_probs(logits, tokens), weights, mask, reduction), src/nn/rl.rs:228-235."""
    return _token_level(capi.LOSS_PG, logits, tokens, mask, reduction, weights=weights)


def clipped_policy_loss(logits, tokens, old_logp, advantages, mask=None, clip=None, reduction=TOKEN_MEAN):
    """clipped_policy_loss (src/nn/rl.rs:265-287) of the tokens' log-probabilities."""
    clip = clip or Clip.symmetric(0.2)
    return _token_level(capi.LOSS_PPO, logits, tokens, mask, reduction, other=old_logp, weights=advantages, clip_low=clip.low, clip_high=clip.high,
                        dual=clip.dual, clamp=clip.log_ratio_clamp)


def kl_estimate(logits, tokens, ref_logp, estimator, delta_clamp=None, mask=None, reduction=TOKEN_MEAN):
    """kl_estimate (src/nn/rl.rs:380-400) of the tokens' log-probabilities."""
    return _token_level(estimator, logits, tokens, mask, reduction, other=ref_logp, clamp=delta_clamp)


def clip_fraction(logp, old_logp, advantages, mask=None, clip=None):
    """clip_fraction (src/nn/rl.rs:293-317), untracked."""
    clip = clip or Clip.symmetric(0.2)
    return ops.clip_fraction(logp, old_logp, advantages, mask=mask, clip_low=clip.low, clip_high=clip.high, dual=clip.dual, clamp=clip.log_ratio_clamp)


def _row_level(which, logits, ref_logits, mask, reduction):
    z = _tempered(logits)
    if len(z.shape) != 4:
        raise ValueError("logits [S, B, T, V]")
    lead = z.shape[:-1]
    ref = None if ref_logits is None else ref_logits.reshape(-1, z.V)
    f = ops.row_forward(z.flat, ref_logits=ref, want_entropy=(which == "entropy"), want_kl=(which == "kl"), want_ref_logp=False, **z.kw())
    raw = (f.kl if which == "kl" else f.entropy).reshape(lead)
    per = raw if mask is None else ops.mask_rows(raw, mask)
    value = ops.reduce_tokens(per, mask, reduction)

    def backward(up):
        d_per = ops.reduce_tokens_backward(lead, mask, reduction, up).reshape(-1)
        kw = dict(g_kl=d_per) if which == "kl" else dict(g_ent=d_per)
        return ops.row_backward(z.flat, f, ref_logits=ref, **kw, **z.kw()).reshape(z.shape)

    return Loss(value, backward)


def categorical_kl(logits, ref_logits, mask=None, reduction=TOKEN_MEAN):
    """categorical_kl (src/nn/rl.rs:327-338). Pass `Tempered(...)` logits for reference_kl."""
    return _row_level("kl", logits, ref_logits, mask, reduction)


def reference_kl(logits, ref_logits, temperature, vocab_mask=None, mask=None, reduction=TOKEN_MEAN):
    """reference_kl (src/nn/rl.rs:347-351): both sides at the sampling temperature, same vocabulary mask."""
    return _row_level("kl", Tempered(logits, temperature, vocab_mask), ref_logits, mask, reduction)


def categorical_entropy(logits, mask=None, reduction=TOKEN_MEAN):
    """categorical_entropy (src/nn/rl.rs:405-414)."""
    return _row_level("entropy", logits, None, mask, reduction)


def _vocab_mask_args(vocab_mask, V):
    """(allow bytes, allow bits) for ops.readout_forward from a bool/uint8 mask [..., V] / [1, V] or
    int32 words of one bit per token [..., ceil(V/32)] / [1, ceil(V/32)]."""
    if vocab_mask is None:
        return None, None
    if vocab_mask.dtype == torch.int32:
        return None, vocab_mask.reshape(-1, vocab_mask.shape[-1]).contiguous()
    allow = vocab_mask.reshape(-1, V)
    return (allow.view(torch.uint8) if allow.dtype == torch.bool else allow).contiguous(), None


def head_token_log_probs(hidden, weight, tokens, round_bf16=False, vocab_mask=None, temperature=1.0):
    """`token_log_probs(head(x), tokens)` and `categorical_entropy(head(x))` per position without the
    logits in between (src/nn/decoder.rs:270-279, then src/nn/rl.rs:134-141, 405-414): `hidden`
    bf16 [..., d], `weight` bf16 [d, V] (the Linear's [in, out] layout), tokens [...]. With
    `vocab_mask` / `temperature` the logits are the tempered ones (src/nn/rl.rs:475-486): what a
    rollout drawn by `head_sample_categorical` under the same mask and temperature is scored with.
    Returns (log-probs [...], entropies [...]). Untracked; needs a compute-capability-10 device."""
    lead = hidden.shape[:-1]
    allow, bits = _vocab_mask_args(vocab_mask, weight.shape[1])
    o = ops.readout_forward(hidden.reshape(-1, hidden.shape[-1]).contiguous(), weight, tokens=tokens.reshape(-1).to(torch.int32).contiguous(), round_bf16=round_bf16, allow=allow, allow_bits=bits,
                            temperature=temperature)
    ops.check_status(o.status)
    return o.logp.reshape(lead), o.entropy.reshape(lead)


def head_sample_categorical(hidden, weight, uniforms, vocab_mask=None, temperature=1.0):
    """`sample_categorical(head(x), temperature, mask, ·)` by inverse CDF against `uniforms` (one per
    position; None or temperature 0: the first maximum) without the logits in between: tokens [...]
    (int32), their log-probs and the per-position entropies (of the tempered distribution).
    `vocab_mask`: a uint8/bool allow-mask [..., V] or [1, V], or int32 words of one bit per token
    [..., ceil(V/32)] or [1, ceil(V/32)]. Refuses a position with no allowed token
    with the reference's message (src/nn/rl.rs:516-519)."""
    lead = hidden.shape[:-1]
    V = weight.shape[1]
    allow, bits = _vocab_mask_args(vocab_mask, V)
    x = hidden.reshape(-1, hidden.shape[-1]).contiguous()
    if not (temperature >= 0.0 and temperature == temperature and temperature != float("inf")):
        raise ValueError("sample_categorical: temperature (must be >= 0)")
    if uniforms is None or temperature == 0.0:
        o = ops.readout_forward(x, weight, greedy=True, allow=allow, allow_bits=bits)
    else:
        o = ops.readout_forward(x, weight, uniforms=uniforms.reshape(-1).contiguous(), allow=allow, allow_bits=bits, temperature=temperature)
    ops.check_status(o.status)
    return o.tokens.reshape(lead), o.logp.reshape(lead), o.entropy.reshape(lead)
