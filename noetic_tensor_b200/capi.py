"""ctypes declarations of the C ABI in include/nrl.h, one to one.

This module is the Python analogue of the `extern "C"` block the noetic-tensor crate would add to
src/tensor/cuda/ffi.rs: structs are laid out exactly as the header's, functions take device
pointers as integers and a stream handle. It raises if libnrl.so is missing: there is no CPU
fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnrl.so")

F32, BF16 = 0, 1
FWD_SAMPLE, FWD_GREEDY, FWD_TOKENS_IN, FWD_MASK_BITS, FWD_ROW_PER_BLOCK = 1, 2, 4, 8, 16
LOSS_PG, LOSS_PPO, LOSS_K1, LOSS_K2, LOSS_K3 = range(5)
REDUCE_NONE, REDUCE_SUM, REDUCE_TOKEN_MEAN, REDUCE_PER_SEQUENCE, REDUCE_SEQUENCE_MEAN = range(5)
E_BAD_ARG, E_UNSUPPORTED, E_WORKSPACE, E_ROW_STATUS, E_NO_DEVICE, E_NOT_FINITE = -1, -2, -3, -4, -5, -6
STATIC_SCRATCH_BYTES = 64 * 1024

u32, u64, f32, f64, ptr = C.c_uint32, C.c_uint64, C.c_float, C.c_double, C.c_uint64


class RowFwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("flags", u32), ("dtype", u32), ("V", u32), ("rows", u64), ("temperature", f32), ("reserved0", u32),
        ("logits", ptr), ("ref_logits", ptr), ("allow_mask", ptr), ("allow_row_stride", u64), ("add_mask", ptr), ("add_row_stride", u64),
        ("uniforms", ptr), ("tokens", ptr), ("logp", ptr), ("ref_logp", ptr), ("kl", ptr), ("entropy", ptr), ("rowstats", ptr), ("status", ptr),
        ("workspace", ptr), ("workspace_bytes", u64),
    ]


class RowBwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("dtype", u32), ("V", u32), ("temperature", f32), ("rows", u64),
        ("logits", ptr), ("ref_logits", ptr), ("allow_mask", ptr), ("allow_row_stride", u64), ("add_mask", ptr), ("add_row_stride", u64),
        ("tokens", ptr), ("rowstats", ptr), ("kl", ptr), ("entropy", ptr), ("g_logp", ptr), ("g_kl", ptr), ("g_ent", ptr), ("d_logits", ptr), ("accumulate", u32), ("mask_bits", u32),
        ("g_uniform", ptr), ("d_ref_logits", ptr),
    ]


class TokenLossArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("kind", u32), ("S", u64), ("B", u64), ("T", u64),
        ("logp", ptr), ("other", ptr), ("weights", ptr), ("weights_per_sequence", u32), ("has_dual", u32), ("mask", ptr),
        ("clip_low", f64), ("clip_high", f64), ("dual", f64), ("clamp", f64), ("has_clamp", u32), ("accumulate", u32),
        ("loss", ptr), ("upstream", ptr), ("dloss_dlogp", ptr),
    ]


class TokenObjectiveArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("reduction", u32), ("policy", TokenLossArgs), ("kl", ptr), ("entropy", ptr),
        ("up_policy", ptr), ("up_kl", ptr), ("up_entropy", ptr), ("out_policy", ptr), ("out_kl", ptr), ("out_entropy", ptr),
        ("g_logp", ptr), ("g_kl", ptr), ("g_ent", ptr),
    ]


class CeArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("V", u32), ("n", u64), ("smoothing", f64),
        ("logp", ptr), ("rowstats", ptr), ("logit_sum", ptr), ("keep", ptr), ("loss", ptr), ("upstream", ptr), ("g_logp", ptr), ("g_uniform", ptr),
    ]


class GumbelArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("dtype", u32), ("V", u32), ("temperature", f32), ("rows", u64),
        ("logits", ptr), ("allow_mask", ptr), ("allow_row_stride", u64), ("add_mask", ptr), ("add_row_stride", u64),
        ("seed", C.c_uint8 * 32), ("word_offset", u64), ("tokens", ptr), ("status", ptr),
    ]


class PackArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("dtype", u32), ("V", u32), ("threads", u32), ("rows", u64),
        ("logits", C.c_void_p), ("ref_logits", C.c_void_p), ("allow_mask", C.c_void_p), ("capacity", u64),
        ("live_words", C.c_void_p), ("row_offset", C.c_void_p), ("packed_logits", C.c_void_p), ("packed_ref", C.c_void_p), ("packed_mask", C.c_void_p),
        ("live_vectors", u64),
    ]


class UnpackArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("dtype", u32), ("V", u32), ("reserved0", u32), ("rows", u64),
        ("live_words", ptr), ("row_offset", ptr), ("packed_logits", ptr), ("packed_ref", ptr), ("packed_mask", ptr),
        ("logits", ptr), ("ref_logits", ptr), ("allow_mask", ptr),
    ]


class LaneArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("op", u32), ("dtype", u32), ("V", u32), ("rows", u64),
        ("x", ptr), ("g", ptr), ("lse", ptr), ("out", ptr), ("out_index", ptr),
    ]


class ReadoutArgs(C.Structure):
    _fields_ = [
        ("struct_size", u32), ("flags", u32), ("V", u32), ("d", u32), ("rows", u64),
        ("hidden", ptr), ("weights", ptr), ("tokens", ptr), ("logp", ptr), ("entropy", ptr), ("rowstats", ptr), ("status", ptr), ("logits_out", ptr),
        ("workspace", ptr), ("workspace_bytes", u64), ("allow_mask", ptr), ("allow_row_stride", u64), ("uniforms", ptr), ("temperature", C.c_float), ("reserved", u32),
    ]


READOUT_W_VD, READOUT_ROUND_BF16, READOUT_ONE_CTA, READOUT_SAMPLE, READOUT_GREEDY, READOUT_MASK_BITS = 1, 2, 4, 8, 16, 32

LANE_SOFTMAX, LANE_LOG_SOFTMAX, LANE_LOGSUMEXP, LANE_ARGMAX, LANE_SUM, LANE_SOFTMAX_BWD, LANE_LOG_SOFTMAX_BWD, LANE_LOGSUMEXP_BWD = range(8)


# every symbol include/nrl.h declares, with its signature
SYMBOLS = {
    "nrl_version": (C.c_int, []),
    "nrl_key": (C.c_char_p, []),
    "nrl_error_string": (C.c_char_p, [C.c_int]),
    "nrl_launch_count": (u64, []),
    "nrl_row_fwd_workspace_bytes": (u64, [u64, u32]),
    "nrl_row_fwd": (C.c_int, [C.POINTER(RowFwdArgs), C.c_void_p]),
    "nrl_row_fwd_static": (C.c_int, [C.POINTER(RowFwdArgs), C.c_void_p]),
    "nrl_row_bwd": (C.c_int, [C.POINTER(RowBwdArgs), C.c_void_p]),
    "nrl_token_loss": (C.c_int, [C.POINTER(TokenLossArgs), C.c_void_p]),
    "nrl_token_objective": (C.c_int, [C.POINTER(TokenObjectiveArgs), C.c_void_p]),
    "nrl_clip_fraction": (C.c_int, [C.POINTER(TokenLossArgs), ptr, C.c_void_p]),
    "nrl_reduce_tokens": (C.c_int, [u32, u64, u64, u64, ptr, ptr, ptr, C.c_void_p]),
    "nrl_reduce_tokens_bwd": (C.c_int, [u32, u64, u64, u64, ptr, ptr, ptr, C.c_void_p]),
    "nrl_reduce_tokens_partial": (C.c_int, [u64, u64, ptr, ptr, ptr, C.c_void_p]),
    "nrl_reduce_tokens_fold": (C.c_int, [u32, u64, u64, ptr, ptr, C.c_void_p]),
    "nrl_reduce_tokens_bwd_pairs": (C.c_int, [u32, u64, u64, u64, u64, u64, ptr, ptr, ptr, ptr, C.c_void_p]),
    "nrl_mask_rows": (C.c_int, [u64, ptr, ptr, ptr, C.c_void_p]),
    "nrl_row_sum": (C.c_int, [u32, u64, u32, ptr, ptr, C.c_void_p]),
    "nrl_ce_tokens": (C.c_int, [C.POINTER(CeArgs), C.c_void_p]),
    "nrl_sample_gumbel": (C.c_int, [C.POINTER(GumbelArgs), C.c_void_p]),
    "nrl_group_advantages": (C.c_int, [u64, u32, u32, C.c_double, u32, ptr, ptr, C.c_void_p]),
    "nrl_lane_op": (C.c_int, [C.POINTER(LaneArgs), C.c_void_p]),
    "nrl_expand_bitmask": (C.c_int, [u64, u32, ptr, u64, ptr, C.c_void_p]),
    "nrl_host_pack_bits": (C.c_int, [u64, u32, C.c_void_p, C.c_void_p, u32]),
    "nrl_host_pack": (C.c_int, [C.POINTER(PackArgs)]),
    "nrl_unpack_rows": (C.c_int, [C.POINTER(UnpackArgs), C.c_void_p]),
    "nrl_readout_workspace_bytes": (u64, [u64, u32, u32, u32]),
    "nrl_readout_fwd": (C.c_int, [C.POINTER(ReadoutArgs), C.c_void_p]),
    "nrl_check_status": (C.c_int, [ptr, u64, C.c_void_p, C.POINTER(u64), C.POINTER(u32)]),
    "nrl_check_scored_finite": (C.c_int, [ptr, ptr, u64, ptr, C.c_void_p, C.POINTER(u64), C.POINTER(f32)]),
}

_lib = None


class NrlError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        msg = lib().nrl_error_string(code).decode() if _lib is not None else str(code)
        super().__init__(f"{what}: {msg} ({code})")


def lib():
    """The loaded libnrl.so. Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m noetic_tensor_b200._build` (nvcc, sm_100a); there is no CPU fallback")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(code, what):
    if code != 0:
        raise NrlError(code, what)
