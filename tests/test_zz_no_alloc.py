"""The forward for callers that cannot allocate device memory (nrl_row_fwd_static).

A serving process that gave all of its device memory to its own arena, or a plugin host that hands
out buffers but no allocator, cannot provide the scratch buffer the split-row forward wants. This
entry point keeps that scratch in a fixed array inside the library instead. The test calls it
through the C ABI twice in a row, on different shapes, and holds every output to the bits of the
ordinary entry point (same kernels, same reduction order), then checks that a shape beyond the
fixed array is refused before anything is launched. It runs last so that a stop-at-first-failure
run has already covered everything else; it also passes on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rows, V, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = (torch.randn(rows, V, generator=g, device=dev) * 3.0).to(torch.bfloat16)
    r = (x.float() + 0.05 * torch.randn(rows, V, generator=g, device=dev)).to(torch.bfloat16)
    allow = (torch.rand(rows, V, generator=g, device=dev) < 0.6).to(torch.uint8)
    allow[:, 0] = 1
    u = torch.rand(rows, generator=g, device=dev)
    return x, r, allow, u


def _args(x, r, allow, u, out):
    from noetic_tensor_b200 import capi

    rows, V = x.shape
    a = capi.RowFwdArgs()
    a.struct_size = C.sizeof(a)
    a.flags, a.dtype, a.V, a.rows, a.temperature = capi.FWD_SAMPLE, capi.BF16, V, rows, 1.0
    a.logits, a.ref_logits, a.allow_mask, a.allow_row_stride, a.uniforms = x.data_ptr(), r.data_ptr(), allow.data_ptr(), V, u.data_ptr()
    for k, t in out.items():
        setattr(a, k, t.data_ptr())
    return a


def _outputs(rows, dev):
    f = lambda *s: torch.full(s, float("nan"), dtype=torch.float32, device=dev)
    return dict(tokens=torch.full((rows,), -7, dtype=torch.int32, device=dev), logp=f(rows), ref_logp=f(rows), kl=f(rows), entropy=f(rows), rowstats=f(rows, 4),
                status=torch.full((rows,), 9, dtype=torch.uint8, device=dev))


def test_static_scratch_forward_matches_the_workspace_forward():
    from noetic_tensor_b200 import capi

    lib = capi.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    # two calls in a row, the second on another shape: what the first left in the array must not matter
    for call, (rows, V) in enumerate([(8, 128256), (12, 32000)]):
        need = lib.nrl_row_fwd_workspace_bytes(rows, V)
        assert 0 < need <= capi.STATIC_SCRATCH_BYTES, "the case must use scratch and fit the fixed array"
        x, r, allow, u = _inputs(rows, V, 100 + call, dev)
        want, got = _outputs(rows, dev), _outputs(rows, dev)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        a = _args(x, r, allow, u, want)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        capi.check(lib.nrl_row_fwd(C.byref(a), stream), "nrl_row_fwd")
        b = _args(x, r, allow, u, got)  # no workspace at all
        capi.check(lib.nrl_row_fwd_static(C.byref(b), stream), "nrl_row_fwd_static")
        torch.cuda.synchronize()
        assert (want["status"] == 0).all()
        for k in want:
            w, g = want[k], got[k]
            if w.dtype == torch.float32:
                w, g = w.view(torch.int32), g.view(torch.int32)
            assert torch.equal(w, g), f"call {call}: {k} differs from nrl_row_fwd"
        tok = got["tokens"].cpu().numpy()
        assert ((tok >= 0) & (tok < V)).all() and allow.cpu().numpy()[np.arange(rows), tok].all()


def test_static_scratch_refuses_shapes_beyond_its_limit():
    from noetic_tensor_b200 import capi

    lib = capi.lib()
    dev = torch.device("cuda:0")
    V = 128256
    rows = max(range(1, 296), key=lambda r: lib.nrl_row_fwd_workspace_bytes(r, V))  # the split shape that needs most
    assert lib.nrl_row_fwd_workspace_bytes(rows, V) > capi.STATIC_SCRATCH_BYTES
    before = lib.nrl_launch_count()
    # the refusal comes before any pointer is touched, so small stand-in buffers are enough
    x = torch.zeros(16, dtype=torch.bfloat16, device=dev)
    a = capi.RowFwdArgs()
    a.struct_size = C.sizeof(a)
    a.dtype, a.V, a.rows, a.temperature, a.logits = capi.BF16, V, rows, 1.0, x.data_ptr()
    rc = lib.nrl_row_fwd_static(C.byref(a), None)
    assert rc == capi.E_WORKSPACE
    assert b"NRL_STATIC_SCRATCH_BYTES" in lib.nrl_error_string(rc)
    assert lib.nrl_launch_count() == before
    # a shape that needs no scratch goes straight through
    rows, V = 512, 1024
    xs, rs, al, u = _inputs(rows, V, 5, dev)
    out = _outputs(rows, dev)
    capi.check(lib.nrl_row_fwd_static(C.byref(_args(xs, rs, al, u, out)), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nrl_row_fwd_static")
    torch.cuda.synchronize()
    assert (out["status"] == 0).all() and torch.isfinite(out["logp"]).all()
