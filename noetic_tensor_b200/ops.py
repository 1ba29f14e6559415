"""Calls into the C ABI with torch tensors as the device buffers.

torch is used for device memory and the current stream only; every computation happens in
libnrl.so. The functions here are thin: they check devices/dtypes, allocate the outputs the C ABI
wants the caller to own, fill the argument struct and launch on torch's current stream.
"""
import ctypes as C

import torch

from . import capi


def _dt(t):
    if t.dtype == torch.float32:
        return capi.F32
    if t.dtype == torch.bfloat16:
        return capi.BF16
    raise TypeError(f"logits must be float32 or bfloat16, got {t.dtype}")


def _p(t):
    return 0 if t is None else t.data_ptr()


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _need(t, dtype, shape, what, dev):
    if t.device != dev or t.dtype != dtype or tuple(t.shape) != tuple(shape) or not t.is_contiguous():
        raise ValueError(f"{what}: expected contiguous {dtype} {tuple(shape)} on {dev}, got {t.dtype} {tuple(t.shape)} on {t.device}")


def _masks(V, rows, allow, add, dev):
    a_stride = d_stride = 0
    if allow is not None:
        allow = allow.view(torch.uint8) if allow.dtype == torch.bool else allow
        if allow.dtype != torch.uint8 or not allow.is_contiguous() or allow.device != dev or allow.numel() not in (V, rows * V):
            raise ValueError("allow mask: contiguous uint8/bool of [rows, V] or [1, V]")
        a_stride = 0 if allow.numel() == V and rows != 1 else V
    if add is not None:
        if add.dtype != torch.float32 or not add.is_contiguous() or add.device != dev or add.numel() not in (V, rows * V):
            raise ValueError("additive mask: contiguous float32 of [rows, V] or [1, V]")
        d_stride = 0 if add.numel() == V and rows != 1 else V
    return allow, a_stride, add, d_stride


def _bit_mask(V, rows, allow_bits, dev):
    """(tensor, stride in words) of a bit-packed allow-mask: int32 [rows, words >= ceil(V/32)] or
    [1, words] (broadcast), bit v of a row = bit (v mod 32) of its word v / 32."""
    if allow_bits.dtype != torch.int32 or allow_bits.dim() != 2 or not allow_bits.is_contiguous() or allow_bits.device != dev:
        raise ValueError(f"allow_bits: contiguous int32 [rows, words] on {dev}")
    if allow_bits.shape[1] < (V + 31) // 32 or allow_bits.shape[0] not in (1, rows):
        raise ValueError("allow_bits: [rows, >= ceil(V/32)] or [1, >= ceil(V/32)]")
    return allow_bits, (0 if allow_bits.shape[0] == 1 and rows != 1 else allow_bits.shape[1])


class RowForward:
    """Outputs of nrl_row_fwd over [rows, V] logits (fields are None when not requested)."""

    __slots__ = ("tokens", "logp", "ref_logp", "kl", "entropy", "rowstats", "status")


def row_forward(logits, *, ref_logits=None, allow=None, add_mask=None, temperature=1.0, uniforms=None, tokens=None, greedy=False,
                want_logp=True, want_entropy=True, want_kl=None, want_ref_logp=None, workspace=None, device=None, allow_bits=None, row_per_block=False):
    """Fused sample / log-prob / KL / entropy over logits [rows, V] (f32 or bf16, CUDA).

    Exactly one of: `uniforms` (sample by inverse CDF), `greedy=True`, `tokens` (given, int32), or
    none (row statistics, entropy and KL only).

    With `device` given, `logits`, `ref_logits` and the masks may be PINNED host tensors: pinned
    memory is mapped into the device's address space, so the kernel reads them in place over the
    host link (with a byte mask, only the mask and the vectors it allows cross it). Everything else
    (uniforms, tokens, the outputs) lives on `device`.

    `allow_bits` instead of `allow`: the mask bit-packed, int32 [rows, ceil(V/32)] (or [1, …]) on
    the device, bit v of a row = bit (v mod 32) of word v / 32; the kernels read V/8 mask bytes
    per row instead of V.

    `row_per_block=True` (NRL_FWD_ROW_PER_BLOCK): the kernel with one thread block per row also
    where the call has enough rows for the grouped kernel."""
    in_dev = logits.device
    dev = torch.device(device) if device is not None else in_dev
    if dev.type != "cuda":
        raise ValueError("row_forward needs CUDA tensors: this library has no CPU path")
    if in_dev.type != "cuda":
        for t in (logits, ref_logits, allow, add_mask):
            if t is not None and t.device != dev and not (t.device.type == "cpu" and t.is_pinned()):
                raise ValueError("row_forward: host inputs must all be pinned (page-locked) tensors")
    if logits.dim() != 2 or not logits.is_contiguous():
        raise ValueError("logits: contiguous [rows, V]")
    rows, V = logits.shape
    a = capi.RowFwdArgs()
    a.struct_size = C.sizeof(a)
    a.dtype, a.V, a.rows, a.temperature = _dt(logits), V, rows, float(temperature)
    a.logits = _p(logits)
    if ref_logits is not None:
        _need(ref_logits, logits.dtype, logits.shape, "ref_logits", in_dev)
        a.ref_logits = _p(ref_logits)
    # with host logits a mask may already be on the device (it is read whole; copying it ahead is cheaper than reading it in place)
    allow, a.allow_row_stride, _, _ = _masks(V, rows, allow, None, dev if (allow is not None and allow.device == dev) else in_dev)
    _, _, add_mask, a.add_row_stride = _masks(V, rows, None, add_mask, dev if (add_mask is not None and add_mask.device == dev) else in_dev)
    a.allow_mask, a.add_mask = _p(allow), _p(add_mask)
    bits_flag = 0
    if allow_bits is not None:
        if allow is not None:
            raise ValueError("give `allow` or `allow_bits`, not both")
        allow_bits, a.allow_row_stride = _bit_mask(V, rows, allow_bits, dev)
        a.allow_mask, bits_flag = _p(allow_bits), capi.FWD_MASK_BITS
    out = RowForward()
    f32 = dict(dtype=torch.float32, device=dev)
    mode = 0
    if uniforms is not None:
        _need(uniforms, torch.float32, (rows,), "uniforms", dev)
        mode, a.uniforms = capi.FWD_SAMPLE, _p(uniforms)
        out.tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    elif greedy:
        mode = capi.FWD_GREEDY
        out.tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    elif tokens is not None:
        _need(tokens, torch.int32, (rows,), "tokens", dev)
        mode = capi.FWD_TOKENS_IN
        out.tokens = tokens
    else:
        out.tokens = None
    a.flags, a.tokens = mode | bits_flag | (capi.FWD_ROW_PER_BLOCK if row_per_block else 0), _p(out.tokens)
    has_ref = ref_logits is not None
    want_kl = has_ref if want_kl is None else want_kl
    want_ref_logp = (has_ref and mode != 0) if want_ref_logp is None else want_ref_logp
    out.logp = torch.empty(rows, **f32) if (want_logp and mode) else None
    out.ref_logp = torch.empty(rows, **f32) if want_ref_logp else None
    out.kl = torch.empty(rows, **f32) if want_kl else None
    out.entropy = torch.empty(rows, **f32) if want_entropy else None
    out.rowstats = torch.empty(rows, 4, **f32)
    out.status = torch.empty(rows, dtype=torch.uint8, device=dev)
    a.logp, a.ref_logp, a.kl, a.entropy, a.rowstats, a.status = _p(out.logp), _p(out.ref_logp), _p(out.kl), _p(out.entropy), _p(out.rowstats), _p(out.status)
    need = capi.lib().nrl_row_fwd_workspace_bytes(rows, V)
    if need:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = _p(workspace), workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_row_fwd(C.byref(a), _stream(dev)), "nrl_row_fwd")
    return out


def row_backward(logits, fwd, *, ref_logits=None, allow=None, add_mask=None, temperature=1.0, g_logp=None, g_kl=None, g_ent=None, out=None, accumulate=False,
                 g_uniform=None, d_ref=None, want_d_logits=True, allow_bits=None):
    """d(logits) [rows, V] f32 from the forward's saved statistics and per-row upstream gradients.
    `g_uniform`: upstream of −mean_v log π_v (label smoothing). `d_ref=True` (or a tensor) also
    returns the KL term's gradient w.r.t. ref_logits, g_kl·(ρ − π): the result is then the pair
    (d_logits or None when `want_d_logits` is False, d_ref_logits)."""
    dev = logits.device
    rows, V = logits.shape
    a = capi.RowBwdArgs()
    a.struct_size = C.sizeof(a)
    a.dtype, a.V, a.rows, a.temperature = _dt(logits), V, rows, float(temperature)
    a.logits, a.ref_logits = _p(logits), _p(ref_logits)
    allow, a.allow_row_stride, add_mask, a.add_row_stride = _masks(V, rows, allow, add_mask, dev)
    a.allow_mask, a.add_mask = _p(allow), _p(add_mask)
    if allow_bits is not None:
        if allow is not None:
            raise ValueError("give `allow` or `allow_bits`, not both")
        allow_bits, a.allow_row_stride = _bit_mask(V, rows, allow_bits, dev)
        a.allow_mask, a.mask_bits = _p(allow_bits), 1
    for name, g in (("g_logp", g_logp), ("g_kl", g_kl), ("g_ent", g_ent), ("g_uniform", g_uniform)):
        if g is not None:
            _need(g, torch.float32, (rows,), name, dev)
    a.tokens, a.rowstats, a.kl, a.entropy = _p(fwd.tokens), _p(fwd.rowstats), _p(fwd.kl), _p(fwd.entropy)
    a.g_logp, a.g_kl, a.g_ent = _p(g_logp), _p(g_kl), _p(g_ent)
    a.g_uniform = _p(g_uniform)
    if not want_d_logits:
        out = None
    elif out is None:
        out = torch.empty(rows, V, dtype=torch.float32, device=dev)
    else:
        _need(out, torch.float32, (rows, V), "d_logits", dev)
    a.d_logits = _p(out)
    if d_ref is True:
        d_ref = torch.empty(rows, V, dtype=torch.float32, device=dev)
    elif d_ref is not None and d_ref is not False:
        _need(d_ref, torch.float32, (rows, V), "d_ref_logits", dev)
    else:
        d_ref = None
    a.d_ref_logits = _p(d_ref)
    a.accumulate = 1 if accumulate else 0
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_row_bwd(C.byref(a), _stream(dev)), "nrl_row_bwd")
    return out if d_ref is None else (out, d_ref)


def _tok_args(kind, logp, other, weights, mask, clip_low=0.0, clip_high=0.0, dual=None, clamp=None):
    S, B, T = logp.shape
    dev = logp.device
    a = capi.TokenLossArgs()
    a.struct_size = C.sizeof(a)
    a.kind, a.S, a.B, a.T = kind, S, B, T
    _need(logp, torch.float32, (S, B, T), "logp", dev)
    a.logp = _p(logp)
    if other is not None:
        _need(other, torch.float32, (S, B, T), "old/ref log-probs", dev)
        a.other = _p(other)
    if weights is not None:
        if weights.dim() == 2:
            _need(weights, torch.float32, (S, B), "weights", dev)
            a.weights_per_sequence = 1
        else:
            _need(weights, torch.float32, (S, B, T), "weights", dev)
        a.weights = _p(weights)
    if mask is not None:
        _need(mask, torch.float32, (S, B, T), "mask", dev)
        a.mask = _p(mask)
    a.clip_low, a.clip_high = clip_low, clip_high
    if dual is not None:
        a.has_dual, a.dual = 1, dual
    if clamp is not None:
        a.has_clamp, a.clamp = 1, clamp
    return a


def token_loss(kind, logp, *, other=None, weights=None, mask=None, clip_low=0.0, clip_high=0.0, dual=None, clamp=None, want_grad=True, upstream=None, accumulate_into=None):
    """Per-token loss [S,B,T] (0 at unscored positions) and upstream · its derivative w.r.t. logp
    (added into `accumulate_into` when that is given: a logp tensor that feeds two losses)."""
    dev = logp.device
    a = _tok_args(kind, logp, other, weights, mask, clip_low, clip_high, dual, clamp)
    if upstream is not None:
        _need(upstream, torch.float32, logp.shape, "upstream", dev)
        a.upstream = _p(upstream)
    loss = torch.empty_like(logp)
    dl = torch.empty_like(logp) if want_grad else None
    if accumulate_into is not None:
        _need(accumulate_into, torch.float32, logp.shape, "accumulate_into", dev)
        dl, a.accumulate = accumulate_into, 1
    a.loss, a.dloss_dlogp = _p(loss), _p(dl)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_token_loss(C.byref(a), _stream(dev)), "nrl_token_loss")
    return loss, dl


class TokenObjective:
    """Outputs of nrl_token_objective: reduced values [S] and per-token gradients [S,B,T] (None when not requested)."""

    __slots__ = ("policy", "kl", "entropy", "g_logp", "g_kl", "g_ent")


def token_objective(kind, logp, reduction, *, other=None, weights=None, mask=None, clip_low=0.0, clip_high=0.0, dual=None, clamp=None, kl=None, entropy=None,
                    up_policy=None, up_kl=None, up_entropy=None, want_grads=True):
    """A token loss of `logp` plus the per-token KL and entropy, all reduced per seed with one
    TokenReduction, and the per-token upstream gradients of the row backward, in one launch
    (nrl_token_objective). `up_*` are the upstream gradients [S] of the three reduced values (None = ones)."""
    dev = logp.device
    S, B, T = logp.shape
    a = capi.TokenObjectiveArgs()
    a.struct_size = C.sizeof(a)
    a.reduction = reduction
    a.policy = _tok_args(kind, logp, other, weights, mask, clip_low, clip_high, dual, clamp)
    out = TokenObjective()
    f32 = dict(dtype=torch.float32, device=dev)
    for name, t in (("kl", kl), ("entropy", entropy)):
        if t is not None:
            _need(t, torch.float32, (S, B, T), name, dev)
    for name, t in (("up_policy", up_policy), ("up_kl", up_kl), ("up_entropy", up_entropy)):
        if t is not None:
            _need(t, torch.float32, (S,), name, dev)
    a.kl, a.entropy = _p(kl), _p(entropy)
    a.up_policy, a.up_kl, a.up_entropy = _p(up_policy), _p(up_kl), _p(up_entropy)
    out.policy = torch.empty(S, **f32)
    out.kl = torch.empty(S, **f32) if kl is not None else None
    out.entropy = torch.empty(S, **f32) if entropy is not None else None
    out.g_logp = torch.empty(S, B, T, **f32) if want_grads else None
    out.g_kl = torch.empty(S, B, T, **f32) if (want_grads and kl is not None) else None
    out.g_ent = torch.empty(S, B, T, **f32) if (want_grads and entropy is not None) else None
    a.out_policy, a.out_kl, a.out_entropy = _p(out.policy), _p(out.kl), _p(out.entropy)
    a.g_logp, a.g_kl, a.g_ent = _p(out.g_logp), _p(out.g_kl), _p(out.g_ent)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_token_objective(C.byref(a), _stream(dev)), "nrl_token_objective")
    return out


def clip_fraction(logp, old_logp, advantages, *, mask=None, clip_low, clip_high, dual=None, clamp=None):
    dev = logp.device
    a = _tok_args(capi.LOSS_PPO, logp, old_logp, advantages, mask, clip_low, clip_high, dual, clamp)
    out = torch.empty(logp.shape[0], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_clip_fraction(C.byref(a), _p(out), _stream(dev)), "nrl_clip_fraction")
    return out


def reduce_tokens(per, mask, reduction):
    S, B, T = per.shape
    dev = per.device
    shape = {capi.REDUCE_NONE: (S, B, T), capi.REDUCE_PER_SEQUENCE: (S, B)}.get(reduction, (S,))
    out = torch.empty(shape, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_reduce_tokens(reduction, S, B, T, _p(per), _p(mask), _p(out), _stream(dev)), "nrl_reduce_tokens")
    return out


def reduce_tokens_backward(shape, mask, reduction, g_out):
    S, B, T = shape
    dev = g_out.device
    d = torch.empty(shape, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_reduce_tokens_bwd(reduction, S, B, T, _p(mask), _p(g_out), _p(d), _stream(dev)), "nrl_reduce_tokens_bwd")
    return d


def mask_rows(x, mask):
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        capi.check(capi.lib().nrl_mask_rows(x.numel(), _p(x), _p(mask), _p(out), _stream(x.device)), "nrl_mask_rows")
    return out


def group_advantages(rewards, *, norm_std=False, eps=0.0, unbiased=True):
    """group_advantages_tensor (src/nn/rl.rs:465-469) over the last axis of f32 rewards [..., N], on the device."""
    if rewards.dtype != torch.float32 or not rewards.is_contiguous() or rewards.device.type != "cuda":
        raise ValueError("rewards: a contiguous float32 CUDA tensor [..., N]")
    n = rewards.shape[-1]
    out = torch.empty_like(rewards)
    with torch.cuda.device(rewards.device):
        capi.check(capi.lib().nrl_group_advantages(rewards.numel() // n, n, int(norm_std), float(eps), int(unbiased), _p(rewards), _p(out), _stream(rewards.device)),
                   "nrl_group_advantages")
    return out


def expand_bitmask(bits, V, rows=None, out=None):
    """U8 allow-mask [rows, V] from bit-packed masks: `bits` int32 [rows, ceil(V/32)] (or [1, …]
    with `rows` given, broadcast), bit v of a row = bit (v mod 32) of word v / 32."""
    dev = bits.device
    if bits.dtype != torch.int32 or bits.dim() != 2 or not bits.is_contiguous() or dev.type != "cuda" or bits.shape[1] < (V + 31) // 32:
        raise ValueError("bits: contiguous int32 CUDA tensor [rows, >= ceil(V/32)]")
    stride = bits.shape[1]
    if rows is None:
        rows = bits.shape[0]
    elif bits.shape[0] == 1 and rows != 1:
        stride = 0
    elif bits.shape[0] != rows:
        raise ValueError("bits: [rows, words] or [1, words]")
    if out is None:
        out = torch.empty(rows, V, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_expand_bitmask(rows, V, _p(bits), stride, _p(out), _stream(dev)), "nrl_expand_bitmask")
    return out


def check_status(status):
    """Raises the reference's error (src/nn/rl.rs:517-519) if any row was refused."""
    bad, bits = C.c_uint64(0), C.c_uint32(0)
    with torch.cuda.device(status.device):
        rc = capi.lib().nrl_check_status(_p(status), status.numel(), _stream(status.device), C.byref(bad), C.byref(bits))
    if rc == capi.E_ROW_STATUS:
        raise RuntimeError(f"sample_categorical: position {bad.value} has no allowed token (every logit −∞ or a NaN)")
    capi.check(rc, "nrl_check_status")


def _rust_float(v):
    """How Rust's `{}` prints a non-finite f64 (the reference's message carries the value)."""
    if v != v:
        return "NaN"
    return "inf" if v > 0 else "-inf"


def check_scored_finite(what, logp, mask=None):
    """`check_scored_finite(what, logp, mask)` (src/nn/rl.rs:204-211): None when every scored
    log-probability (mask != 0; no mask: all) is finite, else the reference's error text, which
    names the first flat position. A host read: it synchronises the stream."""
    dev = logp.device
    if dev.type != "cuda" or logp.dtype != torch.float32 or not logp.is_contiguous():
        raise ValueError("check_scored_finite: a contiguous float32 CUDA tensor")
    if mask is not None:
        _need(mask, torch.float32, logp.shape, "mask", dev)
    result = torch.empty(2, dtype=torch.int64, device=dev)
    pos, val = C.c_uint64(0), C.c_float(0.0)
    with torch.cuda.device(dev):
        rc = capi.lib().nrl_check_scored_finite(_p(logp), _p(mask), logp.numel(), _p(result), _stream(dev), C.byref(pos), C.byref(val))
    if rc == capi.E_NOT_FINITE:
        return f"{what}: the scored log-probability at flat position {pos.value} is {_rust_float(val.value)} (not finite)"
    capi.check(rc, "nrl_check_scored_finite")
    return None


def reduce_tokens_partial(per, mask):
    """Step 1 of a TokenReduction on the sequences this caller holds: `per`, `mask` [n_seq, T] ->
    pairs [n_seq, 2] = (sum of per, sum of mask) per sequence (nrl_reduce_tokens_partial)."""
    n_seq, T = per.shape
    dev = per.device
    _need(per, torch.float32, (n_seq, T), "per", dev)
    if mask is not None:
        _need(mask, torch.float32, (n_seq, T), "mask", dev)
    pairs = torch.empty(n_seq, 2, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_reduce_tokens_partial(n_seq, T, _p(per), _p(mask), _p(pairs), _stream(dev)), "nrl_reduce_tokens_partial")
    return pairs


def reduce_tokens_fold(pairs, S, B, reduction):
    """Step 2: the pairs of all S·B sequences, in sequence order, folded per seed (nrl_reduce_tokens_fold)."""
    dev = pairs.device
    _need(pairs, torch.float32, (S * B, 2), "pairs", dev)
    out = torch.empty((S, B) if reduction == capi.REDUCE_PER_SEQUENCE else (S,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_reduce_tokens_fold(reduction, S, B, _p(pairs), _p(out), _stream(dev)), "nrl_reduce_tokens_fold")
    return out


def reduce_tokens_backward_pairs(reduction, S, B, T, seq_begin, n_seq, pairs, mask, g_out):
    """d_per [n_seq, T] of the local sequences from the whole reduced value's gradient and the
    gathered pairs (nrl_reduce_tokens_bwd_pairs)."""
    dev = g_out.device
    d = torch.empty(n_seq, T, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_reduce_tokens_bwd_pairs(reduction, S, B, T, seq_begin, n_seq, _p(pairs), _p(mask), _p(g_out), _p(d), _stream(dev)), "nrl_reduce_tokens_bwd_pairs")
    return d


class Readout:
    """Outputs of nrl_readout_fwd (fields are None when not requested)."""

    __slots__ = ("logp", "entropy", "rowstats", "status", "logits", "tokens")


def readout_forward(hidden, weights, *, tokens=None, weights_are_vd=False, round_bf16=False, want_logits=False, workspace=None, one_cta=False, uniforms=None, allow=None, greedy=False, temperature=1.0, allow_bits=None):
    """Row statistics of logits = hidden [rows, d] · W without writing the logits (nrl_readout_fwd):
    `hidden` bf16 [rows, d]; `weights` bf16 [d, V] (the reference's Linear layout) or, with
    `weights_are_vd`, [V, d]; `tokens` int32 [rows] (given tokens) for `logp`. `round_bf16` folds
    the logits rounded to bf16; `want_logits` also returns those bf16 logits [rows, V]. With
    `uniforms` (float32 [rows]) the tokens are drawn by inverse CDF instead of given (`tokens` of the
    result), with `greedy` they are each row's first maximum; `allow` is a uint8 allow-mask [rows, V]
    or [1, V], `allow_bits` the same as int32 words [rows, ceil(V/32)] or [1, ceil(V/32)] (bit v of a row =
    bit v mod 32 of word v / 32); `temperature` divides the logits before they are folded (the returned `logits` are the
    undivided ones)."""
    dev = hidden.device
    if dev.type != "cuda":
        raise ValueError("readout_forward needs CUDA tensors: this library has no CPU path")
    rows, d = hidden.shape
    V = weights.shape[0] if weights_are_vd else weights.shape[1]
    _need(hidden, torch.bfloat16, (rows, d), "hidden", dev)
    _need(weights, torch.bfloat16, (V, d) if weights_are_vd else (d, V), "weights", dev)
    a = capi.ReadoutArgs()
    a.struct_size = C.sizeof(a)
    a.flags = (capi.READOUT_W_VD if weights_are_vd else 0) | (capi.READOUT_ROUND_BF16 if round_bf16 else 0) | (capi.READOUT_ONE_CTA if one_cta else 0) | (capi.READOUT_SAMPLE if uniforms is not None else 0) | (capi.READOUT_GREEDY if greedy else 0)
    a.V, a.d, a.rows, a.temperature = V, d, rows, float(temperature)
    a.hidden, a.weights = _p(hidden), _p(weights)
    out = Readout()
    out.logp = out.tokens = None
    if uniforms is not None:
        if tokens is not None or greedy:
            raise ValueError("give one of `tokens`, `uniforms`, `greedy`")
        _need(uniforms, torch.float32, (rows,), "uniforms", dev)
        a.uniforms = _p(uniforms)
        tokens = out.tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    elif greedy:
        if tokens is not None:
            raise ValueError("give `tokens` or `greedy`, not both")
        tokens = out.tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    elif tokens is not None:
        _need(tokens, torch.int32, (rows,), "tokens", dev)
    if tokens is not None:
        a.tokens = _p(tokens)
        out.logp = torch.empty(rows, dtype=torch.float32, device=dev)
    if allow is not None and allow_bits is not None:
        raise ValueError("give `allow` or `allow_bits`, not both")
    if allow is not None:
        allow, a.allow_row_stride, _, _ = _masks(V, rows, allow, None, dev)
        a.allow_mask = _p(allow)
    if allow_bits is not None:
        words = (V + 31) // 32
        if allow_bits.dtype != torch.int32 or allow_bits.dim() != 2 or allow_bits.shape[0] not in (1, rows) or allow_bits.shape[1] < words or allow_bits.device != dev or not allow_bits.is_contiguous():
            raise ValueError("allow_bits: contiguous int32 [rows, >= ceil(V/32)] or [1, ...] on the logits' device")
        a.allow_mask, a.allow_row_stride = _p(allow_bits), (0 if allow_bits.shape[0] == 1 else allow_bits.shape[1])
        a.flags |= capi.READOUT_MASK_BITS
    out.entropy = torch.empty(rows, dtype=torch.float32, device=dev)
    out.rowstats = torch.empty(rows, 4, dtype=torch.float32, device=dev)
    out.status = torch.empty(rows, dtype=torch.uint8, device=dev)
    out.logits = torch.empty(rows, V, dtype=torch.bfloat16, device=dev) if want_logits else None
    a.logp, a.entropy, a.rowstats, a.status, a.logits_out = _p(out.logp), _p(out.entropy), _p(out.rowstats), _p(out.status), _p(out.logits)
    if workspace is None:
        workspace = torch.empty(capi.lib().nrl_readout_workspace_bytes(rows, V, d, a.flags), dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = _p(workspace), workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_readout_fwd(C.byref(a), _stream(dev)), "nrl_readout_fwd")
    return out


def row_sum(logits):
    """Σ_v logits[r, v] per row in f32 (nrl_row_sum)."""
    dev = logits.device
    rows, V = logits.shape
    if not logits.is_contiguous():
        raise ValueError("logits must be contiguous")
    out = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_row_sum(_dt(logits), rows, V, _p(logits), _p(out), _stream(dev)), "nrl_row_sum")
    return out


def ce_tokens(V, logp, *, smoothing=0.0, rowstats=None, logit_sum=None, keep=None, upstream=None, want_loss=True):
    """The O(rows) part of the cross-entropy family (nrl_ce_tokens): returns (loss, g_logp,
    g_uniform), each [n] f32 or None."""
    dev = logp.device
    n = logp.numel()
    a = capi.CeArgs()
    a.struct_size = C.sizeof(a)
    a.V, a.n, a.smoothing = V, n, float(smoothing)
    _need(logp, torch.float32, logp.shape, "logp", dev)
    a.logp, a.rowstats, a.logit_sum, a.keep = _p(logp), _p(rowstats), _p(logit_sum), _p(keep)
    if keep is not None:
        _need(keep, torch.float32, logp.shape, "keep", dev)
    loss = torch.empty_like(logp) if want_loss else None
    g_logp = g_uni = None
    if upstream is not None:
        _need(upstream, torch.float32, logp.shape, "upstream", dev)
        g_logp = torch.empty_like(logp)
        g_uni = torch.empty_like(logp) if smoothing > 0.0 else None
    a.loss, a.upstream, a.g_logp, a.g_uniform = _p(loss), _p(upstream), _p(g_logp), _p(g_uni)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_ce_tokens(C.byref(a), _stream(dev)), "nrl_ce_tokens")
    return loss, g_logp, g_uni


def sample_gumbel(logits, seed, *, word_offset=0, temperature=1.0, allow=None, add_mask=None):
    """The reference's Gumbel-max sampler on the device (nrl_sample_gumbel): `seed` is the 32-byte
    ChaCha20 key, `word_offset` the 32-bit words already drawn. Returns (tokens int32 [rows],
    status uint8 [rows]); the call consumes 2·rows·V words of the stream."""
    dev = logits.device
    rows, V = logits.shape
    if not logits.is_contiguous():
        raise ValueError("logits must be contiguous")
    if len(seed) != 32:
        raise ValueError("seed: 32 bytes")
    a = capi.GumbelArgs()
    a.struct_size = C.sizeof(a)
    a.dtype, a.V, a.rows, a.temperature = _dt(logits), V, rows, float(temperature)
    a.logits = _p(logits)
    allow, a.allow_row_stride, add_mask, a.add_row_stride = _masks(V, rows, allow, add_mask, dev)
    a.allow_mask, a.add_mask = _p(allow), _p(add_mask)
    a.seed[:] = list(seed)
    a.word_offset = int(word_offset)
    tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    status = torch.empty(rows, dtype=torch.uint8, device=dev)
    a.tokens, a.status = _p(tokens), _p(status)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_sample_gumbel(C.byref(a), _stream(dev)), "nrl_sample_gumbel")
    return tokens, status


def _lane(op, x, *, g=None, lse=None, full_out=True, index=False):
    dev = x.device
    if dev.type != "cuda":
        raise ValueError("lane ops run on CUDA tensors only")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous [rows, V] tensor")
    rows, V = x.shape
    a = capi.LaneArgs()
    a.struct_size = C.sizeof(a)
    a.op, a.dtype, a.V, a.rows = op, _dt(x), V, rows
    a.x = _p(x)
    if g is not None:
        _need(g, torch.float32, (rows, V) if op != capi.LANE_LOGSUMEXP_BWD else (rows,), "g", dev)
        a.g = _p(g)
    if lse is not None:
        _need(lse, torch.float32, (rows,), "lse", dev)
        a.lse = _p(lse)
    out = torch.empty((rows, V) if full_out else (rows,), dtype=torch.float32, device=dev)
    a.out = _p(out)
    idx = None
    if index:
        idx = torch.empty(rows, dtype=torch.int32, device=dev)
        a.out_index = _p(idx)
    with torch.cuda.device(dev):
        capi.check(capi.lib().nrl_lane_op(C.byref(a), _stream(dev)), "nrl_lane_op")
    return (idx, out) if index else out


def softmax(x):
    """softmax along the last axis of [rows, V] (src/tensor/activation.rs:15-26), f32 out."""
    return _lane(capi.LANE_SOFTMAX, x)


def log_softmax(x):
    """log_softmax along the last axis (src/tensor/activation.rs:30-42), f32 out."""
    return _lane(capi.LANE_LOG_SOFTMAX, x)


def logsumexp(x):
    """log Σ exp along the last axis with the ±inf rule (src/tensor/activation.rs:71-77), [rows]."""
    return _lane(capi.LANE_LOGSUMEXP, x, full_out=False)


def argmax(x):
    """(index i32 [rows], value f32 [rows]): the first maximum, the first NaN of a row that holds one
    (src/tensor/kernels.rs:184-209)."""
    return _lane(capi.LANE_ARGMAX, x, full_out=False, index=True)


def sum_last(x):
    """Σ along the last axis in the reference's operand order (src/tensor/kernels.rs:122-148)."""
    return _lane(capi.LANE_SUM, x, full_out=False)


def softmax_backward(y, g):
    """y · (g − Σ g·y) from the saved output."""
    return _lane(capi.LANE_SOFTMAX_BWD, y, g=g)


def log_softmax_backward(y, g):
    """g − exp(y) · Σ g from the saved output."""
    return _lane(capi.LANE_LOG_SOFTMAX_BWD, y, g=g)


def logsumexp_backward(x, lse, g):
    """g[row] · exp(x − lse[row])."""
    return _lane(capi.LANE_LOGSUMEXP_BWD, x, g=g, lse=lse)
