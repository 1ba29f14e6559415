"""TEST INFRASTRUCTURE — NOT PRODUCT CODE.

ctypes bindings of the CPU oracle (``liboracle.so``): the restatement of noetic-tensor's
``nn::rl`` path on its ``Cpu(Reference)`` / ``Cpu(Fast)`` arithmetic (f32) and on its F64 path,
plus the random streams and the f64 evaluation of the inverse-CDF sampler. Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may import this
package; the shipped package never does.

The function names and argument meanings follow ``src/nn/rl.rs`` of the reference.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F32, F64, BF16 = 0, 1, 2
NONE, SUM, TOKEN_MEAN, PER_SEQUENCE, SEQUENCE_MEAN = 0, 1, 2, 3, 4
REDUCTIONS = (NONE, SUM, TOKEN_MEAN, PER_SEQUENCE, SEQUENCE_MEAN)
K1, K2, K3 = 1, 2, 3
LOG_RATIO_CLAMP = 20.0  # src/nn/rl.rs:146
KL_DELTA_CLAMP = 20.0  # src/nn/rl.rs:150

OP_TOKEN_LOG_PROBS, OP_PG, OP_PPO, OP_CLIP_FRACTION, OP_KL, OP_REFERENCE_KL, OP_KL_ESTIMATE, OP_ENTROPY = range(8)
# nn::loss (src/nn/loss.rs): `tokens` are the targets; KL_DIV takes pred = logits, target = ref_logits
OP_NLL, OP_CE, OP_MASKED_CE, OP_CE_WITH, OP_KL_DIV = range(8, 13)


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file."""
    srcs = [os.path.join(_HERE, f) for f in ("oracle_api.cpp", "oracle.h", "engine.hpp", "rl.hpp", "loss.hpp", "streams.hpp", "Makefile")]
    if not force and os.path.exists(_LIB_PATH) and all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(s) for s in srcs):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


class _Case(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("op", C.c_int32), ("engine_dtype", C.c_int32), ("reduction", C.c_int32),
        ("S", C.c_int64), ("B", C.c_int64), ("T", C.c_int64), ("V", C.c_int64),
        ("logits", C.c_void_p), ("logits_dtype", C.c_int32), ("ref_dtype", C.c_int32),
        ("ref_logits", C.c_void_p), ("tokens", C.c_void_p), ("logp", C.c_void_p), ("old_logp", C.c_void_p),
        ("ref_logp", C.c_void_p), ("weights", C.c_void_p), ("weights_rank", C.c_int32), ("estimator", C.c_int32),
        ("mask", C.c_void_p), ("vocab_mask", C.c_void_p), ("temperature", C.c_double),
        ("clip_low", C.c_double), ("clip_high", C.c_double), ("dual", C.c_double), ("log_ratio_clamp", C.c_double), ("delta_clamp", C.c_double),
        ("has_dual", C.c_int32), ("has_log_ratio_clamp", C.c_int32), ("has_delta_clamp", C.c_int32), ("vocab_mask_full", C.c_int32),
        ("upstream", C.c_void_p), ("out_value", C.c_void_p), ("out_capacity", C.c_int64), ("out_len", C.c_void_p), ("out_grad", C.c_void_p),
        ("has_ignore_index", C.c_int32), ("reserved0", C.c_int32), ("ignore_index", C.c_int64), ("smoothing", C.c_double), ("out_grad_ref", C.c_void_p),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_last_error.restype = C.c_char_p
        _lib.orc_rl_eval.argtypes = [C.POINTER(_Case)]
    return _lib


def set_backend(fast=False, threads=1):
    """Cpu(Reference) (default) or Cpu(Fast) with `threads` workers (NOETIC_THREADS)."""
    lib().orc_set_backend(int(bool(fast)), int(threads))


class Clip:
    """`nn::rl::Clip` (src/nn/rl.rs:160-198)."""

    def __init__(self, low, high, dual=None, log_ratio_clamp=LOG_RATIO_CLAMP):
        self.low, self.high, self.dual, self.log_ratio_clamp = low, high, dual, log_ratio_clamp

    @staticmethod
    def symmetric(eps):
        return Clip(eps, eps)

    def with_dual(self, c):
        return Clip(self.low, self.high, c, self.log_ratio_clamp)

    def with_log_ratio_clamp(self, b):
        return Clip(self.low, self.high, self.dual, b)


def _storage(a):
    """(array kept alive, dtype code) for logits-sized inputs: float32, float64, or uint16 bf16 bits."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.float32:
        return a, F32
    if a.dtype == np.float64:
        return a, F64
    if a.dtype == np.uint16:
        return a, BF16
    raise TypeError(f"unsupported logits dtype {a.dtype}")


def _f64(a):
    return None if a is None else np.ascontiguousarray(np.asarray(a, dtype=np.float64))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def rl_eval(op, shape, *, dtype=F32, logits=None, ref_logits=None, tokens=None, logp=None, old_logp=None, ref_logp=None, weights=None,
            mask=None, vocab_mask=None, temperature=1.0, clip=None, estimator=K1, delta_clamp=None, reduction=NONE, upstream=None, ignore_index=None, smoothing=0.0, grad_ref=False):
    """Value (float64 array) and, with `upstream`, the gradient of sum(value*upstream) w.r.t. the leaf
    (and, with `grad_ref`, w.r.t. ref_logits as a third result)."""
    S, B, T, V = shape
    n = S * B * T
    keep = []
    c = _Case()
    c.struct_size = C.sizeof(_Case)
    c.op, c.engine_dtype, c.reduction = op, dtype, reduction
    c.S, c.B, c.T, c.V = S, B, T, V
    if logits is not None:
        a, code = _storage(logits)
        assert a.size == n * V
        keep.append(a)
        c.logits, c.logits_dtype = _ptr(a), code
    if ref_logits is not None:
        a, code = _storage(ref_logits)
        assert a.size == n * V
        keep.append(a)
        c.ref_logits, c.ref_dtype = _ptr(a), code
    if tokens is not None:
        a = np.ascontiguousarray(np.asarray(tokens, dtype=np.int64))
        assert a.size == n
        keep.append(a)
        c.tokens = _ptr(a)
    for name, val in (("logp", logp), ("old_logp", old_logp), ("ref_logp", ref_logp), ("mask", mask)):
        if val is not None:
            a = _f64(val)
            assert a.size == n, name
            keep.append(a)
            setattr(c, name, _ptr(a))
    if weights is not None:
        a = _f64(weights)
        keep.append(a)
        c.weights = _ptr(a)
        if a.size == S * B and (a.ndim == 2 or a.size != n):
            c.weights_rank = 2
        else:
            assert a.size == n
            c.weights_rank = 3
    if vocab_mask is not None:
        a = _f64(vocab_mask)
        assert a.size in (V, n * V)
        c.vocab_mask_full = 1 if (a.size == n * V and n != 1) else 0
        keep.append(a)
        c.vocab_mask = _ptr(a)
    c.temperature = float(temperature)
    if clip is not None:
        c.clip_low, c.clip_high = clip.low, clip.high
        c.has_dual, c.dual = (1, clip.dual) if clip.dual is not None else (0, 0.0)
        c.has_log_ratio_clamp, c.log_ratio_clamp = (1, clip.log_ratio_clamp) if clip.log_ratio_clamp is not None else (0, 0.0)
    c.estimator = estimator
    c.has_delta_clamp, c.delta_clamp = (1, delta_clamp) if delta_clamp is not None else (0, 0.0)
    if ignore_index is not None:
        c.has_ignore_index, c.ignore_index = 1, int(ignore_index)
    c.smoothing = float(smoothing)
    cap = max(n, 1)
    out = np.zeros(cap, dtype=np.float64)
    out_len = C.c_int64(0)
    c.out_value, c.out_capacity, c.out_len = _ptr(out), cap, C.cast(C.pointer(out_len), C.c_void_p)
    grad = None
    if upstream is not None:
        up = _f64(upstream)
        keep.append(up)
        c.upstream = _ptr(up)
        grad = np.zeros(n if logp is not None else n * V, dtype=np.float64)
        c.out_grad = _ptr(grad)
        if grad_ref:
            gref = np.zeros(n * V, dtype=np.float64)
            c.out_grad_ref = _ptr(gref)
    rc = lib().orc_rl_eval(C.byref(c))
    if rc != 0:
        raise RuntimeError(lib().orc_last_error().decode())
    value = out[: out_len.value].copy()
    if upstream is not None and grad_ref:
        return value, grad, gref
    return (value, grad) if upstream is not None else value


LANE_SOFTMAX, LANE_LOG_SOFTMAX, LANE_LOGSUMEXP, LANE_ARGMAX, LANE_SUM = range(5)


def lane_op(op, x, *, dtype=F32, upstream=None):
    """softmax / log_softmax / logsumexp / argmax / sum_dim along the last axis of [rows, V] on the
    restated engine (src/tensor/activation.rs:15-42, 71-77; src/tensor/kernels.rs:122-209).
    Returns the value (float64; for argmax a pair (index int64, value)), and with `upstream` also
    the gradient of sum(value * upstream) with respect to x."""
    a, code = _storage(x)
    rows, V = a.shape
    full = op in (LANE_SOFTMAX, LANE_LOG_SOFTMAX)
    value = np.zeros((rows, V) if full else rows, dtype=np.float64)
    index = np.zeros(rows, dtype=np.int64)
    grad = up = None
    if upstream is not None:
        up = _f64(upstream)
        assert up.size == value.size
        grad = np.zeros((rows, V), dtype=np.float64)
    rc = lib().orc_lane_op(op, dtype, _ptr(a), code, C.c_int64(rows), C.c_int64(V), _ptr(up), _ptr(value), _ptr(index), _ptr(grad))
    if rc != 0:
        raise RuntimeError(lib().orc_last_error().decode())
    if op == LANE_ARGMAX:
        return index, value
    return (value, grad) if upstream is not None else value


def out_shape(shape, reduction):
    S, B, T, _ = shape
    return {NONE: (S, B, T), SUM: (S,), TOKEN_MEAN: (S,), PER_SEQUENCE: (S, B), SEQUENCE_MEAN: (S,)}[reduction]


def group_advantages(rewards, n, norm="mean", eps=0.0, unbiased=True):
    """`group_advantages` (src/nn/rl.rs:436-461): norm "mean" is MeanOnly, "std" is Std{eps, unbiased}."""
    r = _f64(rewards).ravel()
    out = np.zeros_like(r)
    rc = lib().orc_group_advantages(_ptr(r), C.c_int64(r.size), C.c_int64(n), 1 if norm == "std" else 0, C.c_double(eps), int(unbiased), _ptr(out))
    if rc != 0:
        raise RuntimeError(lib().orc_last_error().decode())
    return out


def _rust_f64(v):
    """`{}` of an f64 in Rust for the values that matter here."""
    if np.isnan(v):
        return "NaN"
    if np.isinf(v):
        return "inf" if v > 0 else "-inf"
    return repr(float(v))


def check_scored_finite(what, logp, mask=None):
    """`check_scored_finite` (src/nn/rl.rs:204-211): None when every scored log-probability is
    finite, else the reference's error text naming the first flat position."""
    v = _f64(logp).ravel()
    m = None if mask is None else _f64(mask).ravel()
    lib().orc_check_scored_finite.restype = C.c_int64
    i = lib().orc_check_scored_finite(_ptr(v), _ptr(m), C.c_int64(v.size))
    if i < 0:
        return None
    return f"{what}: the scored log-probability at flat position {i} is {_rust_f64(v[i])} (not finite)"


def sha256(data: bytes) -> bytes:
    out = (C.c_uint8 * 32)()
    lib().orc_sha256(data, C.c_int64(len(data)), out)
    return bytes(out)


def derive_seed(root: int, label: str) -> bytes:
    out = (C.c_uint8 * 32)()
    lib().orc_derive_seed(C.c_uint64(root), label.encode(), out)
    return bytes(out)


def chacha20_words(seed: bytes, n: int, skip: int = 0):
    assert len(seed) == 32
    out = np.zeros(n, dtype=np.uint32)
    lib().orc_chacha20_words((C.c_uint8 * 32).from_buffer_copy(seed), C.c_int64(skip), C.c_int64(n), _ptr(out))
    return out


def row_uniforms(root: int, label: str, rows: int):
    out = np.zeros(rows, dtype=np.float32)
    lib().orc_row_uniforms(C.c_uint64(root), label.encode(), C.c_int64(rows), _ptr(out))
    return out


def bf16_from_f32(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(x.shape, dtype=np.uint16)
    lib().orc_bf16_from_f32(_ptr(x), C.c_int64(x.size), _ptr(out))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.zeros(x.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(_ptr(x), C.c_int64(x.size), _ptr(out))
    return out


def _masks(rows, V, add_mask, allow):
    am = ast = al = alst = None
    if add_mask is not None:
        am = np.ascontiguousarray(add_mask, dtype=np.float32).reshape(-1, V)
        ast = 0 if am.shape[0] == 1 else V
        assert am.shape[0] in (1, rows)
    if allow is not None:
        al = np.ascontiguousarray(allow, dtype=np.uint8).reshape(-1, V)
        alst = 0 if al.shape[0] == 1 else V
        assert al.shape[0] in (1, rows)
    return am, ast or 0, al, alst or 0


def sample_gumbel(logits, temperature, root, label, add_mask=None, allow=None):
    """The reference's `sample_categorical` (src/nn/rl.rs:510-529) on [rows, V] logits."""
    a, code = _storage(logits)
    rows, V = a.shape
    am, ast, al, alst = _masks(rows, V, add_mask, allow)
    tok = np.zeros(rows, dtype=np.int64)
    bad = C.c_int64(-1)
    rc = lib().orc_sample_gumbel(_ptr(a), code, C.c_int64(rows), C.c_int64(V), C.c_double(temperature), _ptr(am), C.c_int64(ast), _ptr(al), C.c_int64(alst),
                                 C.c_uint64(root), label.encode(), _ptr(tok), C.byref(bad))
    if rc != 0:
        raise RuntimeError(f"sample_categorical: position {bad.value} has no allowed token (every logit −∞ or a NaN)")
    return tok


def sample_inverse_cdf(logits, temperature=1.0, uniforms=None, ref_logits=None, add_mask=None, allow=None, given_tokens=None):
    """f64 evaluation of the inverse-CDF sampler and the per-row quantities on [rows, V] logits.

    Returns a dict: tokens (int64, −1 on a refused row), boundary (uint8), logp, ref_logp, kl,
    entropy (float64) and status (uint8; bit0 no allowed token, bit1 NaN)."""
    a, code = _storage(logits)
    rows, V = a.shape
    r = rcode = None
    if ref_logits is not None:
        r, rcode = _storage(ref_logits)
        assert r.shape == a.shape
    am, ast, al, alst = _masks(rows, V, add_mask, allow)
    u = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
    gt = None if given_tokens is None else np.ascontiguousarray(given_tokens, dtype=np.int64)
    if gt is None and temperature != 0.0:
        assert u is not None and u.size == rows
    o = dict(tokens=np.zeros(rows, np.int64), boundary=np.zeros(rows, np.uint8), logp=np.zeros(rows), ref_logp=np.zeros(rows), kl=np.zeros(rows),
             entropy=np.zeros(rows), status=np.zeros(rows, np.uint8))
    lib().orc_sample_inverse_cdf(_ptr(a), code, _ptr(r), rcode or 0, C.c_int64(rows), C.c_int64(V), C.c_double(temperature), _ptr(am), C.c_int64(ast),
                                 _ptr(al), C.c_int64(alst), _ptr(u), _ptr(gt), _ptr(o["tokens"]), _ptr(o["boundary"]), _ptr(o["logp"]),
                                 _ptr(o["ref_logp"]) if r is not None else None, _ptr(o["kl"]) if r is not None else None, _ptr(o["entropy"]), _ptr(o["status"]))
    if r is None:
        o["ref_logp"] = o["kl"] = None
    return o
