"""CPU checks of the C-ABI boundary: the library builds, loads, exports every symbol that
include/nrl.h declares, and the ctypes structs have the sizes the header's layout implies."""
import ctypes as C
import os
import re

from noetic_tensor_b200 import _build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "nrl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(nrl_[a-z0-9_]+)\s*\(", text))


def test_library_builds_and_exports_every_declared_symbol():
    _build.build()
    l = capi.lib()
    declared = header_functions()
    assert declared == set(capi.SYMBOLS), (declared ^ set(capi.SYMBOLS))
    for name in declared:
        assert hasattr(l, name), name


def test_identity_calls_need_no_gpu():
    l = capi.lib()
    assert l.nrl_version() >= 100
    key = l.nrl_key().decode()
    assert key.startswith("cuda-sm100a-") and key.endswith(_build.source_hash())
    assert b"bad argument" in l.nrl_error_string(capi.E_BAD_ARG)
    assert l.nrl_launch_count() == 0 or l.nrl_launch_count() > 0


def test_struct_layouts():
    # sizes follow from the header's field lists (8-byte alignment, no packing)
    assert C.sizeof(capi.RowFwdArgs) == 4 * 4 + 8 + 4 + 4 + 16 * 8
    assert C.sizeof(capi.RowBwdArgs) == 4 * 4 + 8 + 14 * 8 + 8 + 2 * 8
    assert C.sizeof(capi.TokenLossArgs) == 8 + 3 * 8 + 3 * 8 + 8 + 8 + 4 * 8 + 8 + 3 * 8
    assert C.sizeof(capi.CeArgs) == 8 + 8 + 8 + 8 * 8
    assert C.sizeof(capi.GumbelArgs) == 4 * 4 + 8 + 5 * 8 + 32 + 8 + 2 * 8
    assert C.sizeof(capi.LaneArgs) == 4 * 4 + 8 + 5 * 8
    assert C.sizeof(capi.PackArgs) == 4 * 4 + 8 + 3 * 8 + 8 + 5 * 8 + 8
    assert C.sizeof(capi.UnpackArgs) == 4 * 4 + 8 + 8 * 8
    assert C.sizeof(capi.ReadoutArgs) == 4 * 4 + 8 + 9 * 8 + 8 + 3 * 8 + 4 + 4
    assert C.sizeof(capi.TokenObjectiveArgs) == 8 + C.sizeof(capi.TokenLossArgs) + 11 * 8


def test_argument_checks_run_before_any_cuda_call():
    l = capi.lib()
    a = capi.RowFwdArgs()
    assert l.nrl_row_fwd(C.byref(a), None) == capi.E_BAD_ARG  # struct_size 0
    a.struct_size = C.sizeof(a)
    assert l.nrl_row_fwd(C.byref(a), None) == capi.E_BAD_ARG  # no rows, no logits
    a.rows, a.V, a.logits, a.temperature, a.dtype = 4, 16, 256, 1.0, 7
    assert l.nrl_row_fwd(C.byref(a), None) == capi.E_UNSUPPORTED
    a.dtype, a.flags = capi.F32, capi.FWD_SAMPLE | capi.FWD_GREEDY
    assert l.nrl_row_fwd(C.byref(a), None) == capi.E_BAD_ARG
    a.flags, a.temperature = 0, 0.0
    assert l.nrl_row_fwd(C.byref(a), None) == capi.E_BAD_ARG
    # few long rows are split over several blocks and need scratch; many rows do not
    assert l.nrl_row_fwd_workspace_bytes(262144, 128256) == 0
    assert l.nrl_row_fwd_workspace_bytes(32, 128256) > 0
    assert l.nrl_row_fwd_workspace_bytes(32, 16) == 0
    # the cross-entropy entries
    assert l.nrl_row_sum(capi.F32, 0, 16, 256, 256, None) == capi.E_BAD_ARG
    assert l.nrl_row_sum(9, 4, 16, 256, 256, None) == capi.E_UNSUPPORTED
    c = capi.CeArgs()
    c.struct_size, c.V, c.n, c.logp, c.loss, c.smoothing = C.sizeof(c), 16, 4, 256, 256, 1.5
    assert l.nrl_ce_tokens(C.byref(c), None) == capi.E_BAD_ARG  # label smoothing outside [0, 1]
    c.smoothing = 0.1
    assert l.nrl_ce_tokens(C.byref(c), None) == capi.E_BAD_ARG  # smoothing needs rowstats and the logit sums
    b = capi.RowBwdArgs()
    b.struct_size, b.rows, b.V, b.logits, b.temperature, b.dtype, b.rowstats = C.sizeof(b), 4, 16, 256, 1.0, capi.F32, 256
    assert l.nrl_row_bwd(C.byref(b), None) == capi.E_BAD_ARG  # no output
    b.d_logits, b.g_uniform, b.allow_mask, b.allow_row_stride = 256, 256, 256, 16
    assert l.nrl_row_bwd(C.byref(b), None) == capi.E_UNSUPPORTED  # label smoothing under a vocabulary mask
