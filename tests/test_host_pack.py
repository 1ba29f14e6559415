"""nrl_host_pack is host code (no CUDA call): what it keeps of byte-masked rows is checked here
on the CPU against numpy, for bf16 and f32 storage, with and without a reference stream, several
thread counts, ragged word counts and the capacity refusal. The device side (nrl_unpack_rows and
the packed host path end to end) is in test_gpu_hostpath.py."""
import ctypes as C

import numpy as np
import pytest

from noetic_tensor_b200 import capi


def pack(x, r, m, threads, capacity):
    rows, V = m.shape
    words = (V // 8 + 63) // 64
    esize = x.dtype.itemsize
    live_words = np.zeros((rows, words), np.uint64)
    row_offset = np.zeros(rows + 1, np.uint32)
    pl = np.zeros((capacity, 8), x.dtype)
    pr = np.zeros((capacity, 8), x.dtype) if r is not None else None
    pm = np.zeros(capacity, np.uint64)
    a = capi.PackArgs()
    a.struct_size = C.sizeof(a)
    a.dtype = capi.F32 if esize == 4 else capi.BF16
    a.V, a.threads, a.rows, a.capacity = V, threads, rows, capacity
    p = lambda t: None if t is None else t.ctypes.data_as(C.c_void_p)
    a.logits, a.ref_logits, a.allow_mask = p(x), p(r), p(m)
    a.live_words, a.row_offset, a.packed_logits, a.packed_ref, a.packed_mask = p(live_words), p(row_offset), p(pl), p(pr), p(pm)
    rc = capi.lib().nrl_host_pack(C.byref(a))
    return rc, int(a.live_vectors), live_words, row_offset, pl, pr, pm


@pytest.mark.parametrize("V", [8, 64, 520, 4104, 128256])
@pytest.mark.parametrize("dtype,ref", [(np.uint16, True), (np.float32, False), (np.float32, True)])
def test_pack_keeps_exactly_the_live_vectors(V, dtype, ref):
    g = np.random.default_rng(V)
    rows = 9 if V > 10000 else 37
    x = g.integers(0, 60000, (rows, V)).astype(dtype) if dtype == np.uint16 else g.normal(0, 1, (rows, V)).astype(np.float32)
    r = (x + 1).astype(dtype) if ref else None
    m = (g.uniform(0, 1, (rows, V)) < 0.02).astype(np.uint8)
    m[:, : min(V, 256)] |= (g.uniform(0, 1, (rows, min(V, 256))) < 0.5).astype(np.uint8)
    m[3] = 0  # a row with nothing allowed
    live = m.reshape(rows, V // 8, 8).any(axis=2)
    total = int(live.sum())
    for threads in (1, 3, 16):
        rc, n, words, off, pl, pr, pm = pack(x, r, m, threads, total + 5)
        assert rc == 0 and n == total
        assert np.array_equal(off, np.concatenate([[0], np.cumsum(live.sum(axis=1))]).astype(np.uint32))
        bits = np.unpackbits(words.view(np.uint8).reshape(rows, -1), axis=1, bitorder="little")[:, : V // 8].astype(bool)
        assert np.array_equal(bits, live)
        assert np.array_equal(pl[:n], x.reshape(rows, V // 8, 8)[live])
        if ref:
            assert np.array_equal(pr[:n], r.reshape(rows, V // 8, 8)[live])
        assert np.array_equal(pm[:n].view(np.uint8).reshape(n, 8), m.reshape(rows, V // 8, 8)[live])
    rc, n, *_ = pack(x, r, m, 4, max(total - 1, 0))
    assert rc == capi.E_WORKSPACE and n == total, "too small a capacity is refused and the need reported"


def test_pack_argument_checks():
    a = capi.PackArgs()
    assert capi.lib().nrl_host_pack(C.byref(a)) == capi.E_BAD_ARG
    a.struct_size, a.rows, a.V = C.sizeof(a), 1, 12  # V not a multiple of 8
    assert capi.lib().nrl_host_pack(C.byref(a)) == capi.E_BAD_ARG


@pytest.mark.parametrize("V", [1, 31, 32, 33, 100, 4104, 128256])
def test_pack_bits_on_the_host(V):
    """nrl_host_pack_bits: bit v of a row = bit v mod 32 of word v / 32, any non-zero byte allowed."""
    g = np.random.default_rng(V)
    rows = 5 if V > 10000 else 23
    m = (g.uniform(0, 1, (rows, V)) < 0.3).astype(np.uint8) * g.integers(1, 255, (rows, V)).astype(np.uint8)
    words = (V + 31) // 32
    want = np.packbits(np.pad(m != 0, ((0, 0), (0, (-V) % 32))), axis=1, bitorder="little").view(np.uint32)
    for threads in (1, 3, 16):
        bits = np.full((rows, words), 0xFFFFFFFF, np.uint32)
        rc = capi.lib().nrl_host_pack_bits(rows, V, m.ctypes.data_as(C.c_void_p), bits.ctypes.data_as(C.c_void_p), threads)
        assert rc == 0 and np.array_equal(bits, want)
    assert capi.lib().nrl_host_pack_bits(0, V, None, None, 1) == capi.E_BAD_ARG


def test_pack_after_fork():
    """The packers keep worker threads between calls. A forked child inherits the pool object but
    not its threads: it must start its own and leave cleanly, and the parent's must go on working."""
    import os
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    script = r"""
import os, sys
import numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r)
from test_host_pack import pack
g = np.random.default_rng(0); rows, V = 64, 4104
x = g.integers(0, 60000, (rows, V)).astype(np.uint16); m = (g.uniform(0, 1, (rows, V)) < 0.05).astype(np.uint8)
live = int(m.reshape(rows, V // 8, 8).any(axis=2).sum())
assert pack(x, None, m, 4, live + 1)[1] == live
pid = os.fork()
if pid == 0:
    os._exit(0 if pack(x, None, m, 4, live + 1)[1] == live else 1)
_, st = os.waitpid(pid, 0)
assert os.WIFEXITED(st) and os.WEXITSTATUS(st) == 0, st
assert pack(x, None, m, 4, live + 1)[1] == live
print("ok")
""" % (here, os.path.dirname(here))
    r = subprocess.run([sys.executable, "-W", "ignore", "-c", script], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-2000:]
