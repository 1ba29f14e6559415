"""Rows that live in host memory: nrl_unpack_rows against numpy, and the packed host path
(hostpath.HostForward) end to end against the resident forward on the same rows.

The packed path uploads only the vectors a byte mask allows and leaves the rest of the device
buffers as they were, so the slots are poisoned with NaN bit patterns first: every result must
still be bit-equal to the forward over the rows uploaded whole.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int32) if t.dtype == torch.float32 else t


def _unpack(dev, dtype, V, rows, words, off, pl, pr, pm, poison):
    from noetic_tensor_b200 import capi

    x = torch.full((rows, V), poison, dtype=dtype, device=dev)
    r = torch.full((rows, V), poison, dtype=dtype, device=dev) if pr is not None else None
    m = torch.full((rows, V), 7, dtype=torch.uint8, device=dev)
    a = capi.UnpackArgs()
    a.struct_size = C.sizeof(a)
    a.dtype, a.V, a.rows = (capi.F32 if dtype == torch.float32 else capi.BF16), V, rows
    a.live_words, a.row_offset = words.data_ptr(), off.data_ptr()
    a.packed_logits, a.packed_mask = pl.data_ptr(), pm.data_ptr()
    a.packed_ref = pr.data_ptr() if pr is not None else 0
    a.logits, a.allow_mask = x.data_ptr(), m.data_ptr()
    a.ref_logits = r.data_ptr() if r is not None else 0
    capi.check(capi.lib().nrl_unpack_rows(C.byref(a), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "nrl_unpack_rows")
    torch.cuda.synchronize(dev)
    return x, r, m


@pytest.mark.parametrize("V", [8, 72, 520, 4104, 128256])
@pytest.mark.parametrize("dtype,ref", [(torch.bfloat16, True), (torch.float32, True), (torch.bfloat16, False)])
def test_unpack_puts_live_vectors_in_place(V, dtype, ref):
    from test_host_pack import pack

    dev = torch.device("cuda:0")
    g = np.random.default_rng(V + 1)
    rows = 7 if V > 10000 else 41
    npdt = np.uint16 if dtype == torch.bfloat16 else np.float32
    x = g.integers(0, 0x7f00, (rows, V)).astype(npdt) if npdt == np.uint16 else g.normal(0, 1, (rows, V)).astype(np.float32)
    r = (x + 1).astype(npdt) if ref else None
    m = (g.uniform(0, 1, (rows, V)) < 0.03).astype(np.uint8) * g.integers(1, 255, (rows, V)).astype(np.uint8)
    m[2] = 0
    live = m.reshape(rows, V // 8, 8).any(axis=2)
    rc, n, words, off, pl, pr, pm = pack(x, r, m, 4, int(live.sum()) + 3)
    assert rc == 0

    def up(a, dt):
        return None if a is None else torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(dev).view(dt)

    xd, rd, md = _unpack(dev, dtype, V, rows, torch.from_numpy(words.view(np.int64)).to(dev), torch.from_numpy(off.view(np.int32)).to(dev),
                         up(pl, dtype), up(pr, dtype), torch.from_numpy(pm.view(np.int64)).to(dev), float("nan"))
    assert np.array_equal(md.cpu().numpy(), m), "the byte mask is written in full"
    elem = np.repeat(live, 8, axis=1)
    back = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16) if dtype == torch.bfloat16 else t.cpu().numpy()
    assert np.array_equal(back(xd)[elem], x[elem])
    assert np.isnan(xd.float().cpu().numpy()[~elem]).all(), "vectors that are not live are left as they were"
    if ref:
        assert np.array_equal(back(rd)[elem], r[elem])


@pytest.mark.parametrize("dtype,ref,rows,chunk", [(torch.bfloat16, True, 1300, 512), (torch.bfloat16, False, 700, 256), (torch.float32, True, 300, 128)])
def test_packed_host_path_equals_resident_forward(dtype, ref, rows, chunk):
    """Grammar masks at the Llama-3 vocabulary: a full chunk, ragged last chunks that take the
    split-row kernels, with the device slots poisoned beforehand."""
    from noetic_tensor_b200 import ops, synth
    from noetic_tensor_b200.hostpath import HostForward

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    V = 128256 if dtype == torch.bfloat16 else 32000
    x = synth.normal_logits(rows, V, 3.0, dtype, gen, dev)
    r = synth.perturbed(x, 0.05, gen) if ref else None
    m = synth.grammar_masks(rows, V, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    # the kernel (and with it the rounding of the merges) is chosen by the number of rows in a
    # launch, so the resident forward is run over the same row chunks
    parts = [ops.row_forward(x[a:a + chunk], ref_logits=None if r is None else r[a:a + chunk], allow=m[a:a + chunk], uniforms=u[a:a + chunk]) for a in range(0, rows, chunk)]
    want = {n: torch.cat([getattr(f, n) for f in parts]).cpu() for n in ("tokens", "logp", "entropy") + (("kl",) if ref else ())}
    pin = lambda t: None if t is None else t.cpu().pin_memory()
    hx, hr, hm, hu = pin(x), pin(r), pin(m), pin(u)
    for packed in (True, False):
        hf = HostForward(V, dtype, chunk_rows=chunk, ref=ref, mask=True, device=dev, packed=packed, threads=4)
        for s in hf.slots:
            s["x"].fill_(float("nan"))
            if ref:
                s["r"].fill_(float("nan"))
        for again in range(2):  # the second call reuses slots that hold the first call's rows
            got = hf.run(hx, hu, ref=hr, mask=hm)
            for name in ("tokens", "logp", "entropy") + (("kl",) if ref else ()):
                assert torch.equal(_bits(got[name]), _bits(want[name])), (name, packed, again)
            assert (got["status"] == 0).all()
        if packed:
            assert hf.packed_chunks > 0 and hf.whole_chunks == 0
            assert hf.h2d_bytes < 0.5 * rows * hf.bytes_per_row()[0], "the link carries the live vectors only"
        else:
            assert hf.packed_chunks == 0


def test_chunk_that_outgrows_staging_is_uploaded_whole():
    from noetic_tensor_b200 import ops, synth
    from noetic_tensor_b200.hostpath import HostForward

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    rows, V = 96, 4096
    x = synth.normal_logits(rows, V, 2.0, torch.bfloat16, gen, dev)
    m = (torch.rand(rows, V, generator=gen, device=dev) < 0.5).to(torch.uint8)  # every vector live
    u = synth.uniforms(rows, gen, dev)
    parts = [ops.row_forward(x[a:a + 32], allow=m[a:a + 32], uniforms=u[a:a + 32]) for a in range(0, rows, 32)]  # the same launches
    hf = HostForward(V, torch.bfloat16, chunk_rows=32, ref=False, mask=True, device=dev, live_fraction=0.25, threads=2)
    got = hf.run(x.cpu().pin_memory(), u.cpu().pin_memory(), mask=m.cpu().pin_memory())
    assert hf.whole_chunks == 3 and hf.packed_chunks == 0
    assert torch.equal(got["tokens"], torch.cat([f.tokens for f in parts]).cpu())
    assert torch.equal(_bits(got["logp"]), _bits(torch.cat([f.logp for f in parts]).cpu()))


@pytest.mark.parametrize("dtype,ref,rows", [(torch.bfloat16, True, 1300), (torch.bfloat16, False, 300), (torch.float32, True, 40)])
def test_mapped_host_rows_equal_the_resident_forward(dtype, ref, rows):
    """The forward reading pinned host memory in place (no staging copy): the same launch shape as
    the resident call, so every result is bit-equal."""
    from noetic_tensor_b200 import ops, synth
    from noetic_tensor_b200.hostpath import HostForward

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(13)
    V = 128256 if dtype == torch.bfloat16 else 32000
    x = synth.normal_logits(rows, V, 3.0, dtype, gen, dev)
    r = synth.perturbed(x, 0.05, gen) if ref else None
    m = synth.grammar_masks(rows, V, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    want = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    pin = lambda t: None if t is None else t.cpu().pin_memory()
    hf = HostForward(V, dtype, chunk_rows=64, ref=ref, mask=True, device=dev, packed=False)
    hx, hu, hr, hm = pin(x), pin(u), pin(r), pin(m)
    for by_copy in (False, True):  # everything in place; the mask by copies (one chunk: the same launch shape)
        got = hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=rows, mask_by_copy=by_copy)
        for name in ("tokens", "logp", "entropy") + (("kl",) if ref else ()):
            assert torch.equal(_bits(got[name]), _bits(getattr(want, name).cpu())), (name, by_copy)
        assert (got["status"] == 0).all()
    # several chunks, the mask one chunk ahead: the launches of the resident forward over the same chunks
    chunk = max(16, rows // 3)
    got = hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=chunk)
    bits = torch.from_numpy(np.packbits(np.pad(m.cpu().numpy(), ((0, 0), (0, (-V) % 32))), axis=1, bitorder="little").view(np.int32)).pin_memory()
    got_bits = hf.run_mapped(hx, hu, ref=hr, mask_bits=bits, chunk_rows=chunk)  # the same rows with bit-packed masks
    for name in ("tokens", "logp", "entropy"):
        assert torch.equal(_bits(got_bits[name]), _bits(got[name])), name
    parts = [ops.row_forward(x[a:a + chunk], ref_logits=None if r is None else r[a:a + chunk], allow=m[a:a + chunk], uniforms=u[a:a + chunk]) for a in range(0, rows, chunk)]
    for name in ("tokens", "logp", "entropy") + (("kl",) if ref else ()):
        assert torch.equal(_bits(got[name]), _bits(torch.cat([getattr(f, name) for f in parts]).cpu())), name
    # the byte mask packed into bits by host threads, chunk by chunk: the byte mask's results
    got_hb = hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=chunk, pack_bits_on_host=True)
    for name in ("tokens", "logp", "entropy"):
        assert torch.equal(_bits(got_hb[name]), _bits(got[name])), ("host-packed bits", name)
    # a smaller first chunk (its mask copy is the exposed one): the same launches, resident
    first = max(8, chunk // 4)
    got = hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=chunk, first_chunk_rows=first)
    cuts = [0] + list(range(first, rows, chunk)) + [rows]
    parts = [ops.row_forward(x[a:b], ref_logits=None if r is None else r[a:b], allow=m[a:b], uniforms=u[a:b]) for a, b in zip(cuts[:-1], cuts[1:])]
    for name in ("tokens", "logp", "entropy"):
        assert torch.equal(_bits(got[name]), _bits(torch.cat([getattr(f, name) for f in parts]).cpu())), ("first chunk", name)
    with pytest.raises(ValueError, match="pinned"):
        ops.row_forward(x.cpu(), allow=pin(m), uniforms=u, device=dev)


def test_hybrid_host_path_is_its_two_halves():
    """run_hybrid: a share of the rows through the mapped path and the rest through the packed
    path at the same time, on two threads and two streams: the bits of the two paths run one after
    the other on the same shares, and the resident forward's values."""
    from noetic_tensor_b200 import ops, synth
    from noetic_tensor_b200.hostpath import HostForward

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(21)
    V, rows, chunk = 128256, 1400, 128
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev)
    r = synth.perturbed(x, 0.05, gen)
    m = synth.grammar_masks(rows, V, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    pin = lambda t: t.cpu().pin_memory()
    hx, hu, hr, hm = pin(x), pin(u), pin(r), pin(m)
    hf = HostForward(V, torch.bfloat16, chunk_rows=chunk, device=dev, threads=4)
    got = hf.run_hybrid(hx, hu, ref=hr, mask=hm, packed_share=0.4, mapped_chunk_rows=300, packed_threads=2)
    n_packed = int(rows * 0.4) // chunk * chunk
    n_mapped = rows - n_packed
    first = hf.run_mapped(hx[:n_mapped], hu[:n_mapped], ref=hr[:n_mapped], mask=hm[:n_mapped], chunk_rows=300, first_chunk_rows=300, pack_bits_on_host=True)
    second = HostForward(V, torch.bfloat16, chunk_rows=chunk, device=dev, threads=2).run(hx[n_mapped:], hu[n_mapped:], ref=hr[n_mapped:], mask=hm[n_mapped:])
    for name in ("tokens", "logp", "kl", "entropy", "status"):
        assert torch.equal(_bits(got[name][:n_mapped]), _bits(first[name])), ("mapped share", name)
        assert torch.equal(_bits(got[name][n_mapped:]), _bits(second[name])), ("packed share", name)
    want = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    assert int((got["tokens"] != want.tokens.cpu()).sum()) <= 2
    same = got["tokens"] == want.tokens.cpu()
    assert torch.allclose(got["logp"][same], want.logp.cpu()[same], rtol=1e-5, atol=1e-6) and torch.allclose(got["entropy"], want.entropy.cpu(), rtol=1e-5, atol=1e-6)
    assert torch.allclose(got["kl"], want.kl.cpu(), rtol=1e-5, atol=1e-6)
    again = hf.run_hybrid(hx, hu, ref=hr, mask=hm, packed_share=0.4, mapped_chunk_rows=300, packed_threads=2)
    for name in ("tokens", "logp", "kl", "entropy"):
        assert torch.equal(_bits(again[name]), _bits(got[name])), ("run to run", name)


@pytest.mark.parametrize("V", [1, 7, 8, 31, 32, 33, 100, 4104, 128256])
def test_expand_bitmask(V):
    from noetic_tensor_b200 import ops

    dev = torch.device("cuda:0")
    g = np.random.default_rng(V)
    rows = 5
    m = (g.uniform(0, 1, (rows, V)) < 0.3).astype(np.uint8)
    words = (V + 31) // 32
    padded = np.zeros((rows, words * 32), np.uint8)
    padded[:, :V] = m
    bits = np.packbits(padded, axis=1, bitorder="little").view(np.uint32).astype(np.int64)
    bits = torch.from_numpy(bits.astype(np.uint32).view(np.int32).reshape(rows, words)).to(dev)
    out = ops.expand_bitmask(bits, V)
    assert np.array_equal(out.cpu().numpy(), m)
    one = ops.expand_bitmask(bits[:1].contiguous(), V, rows=4)
    assert np.array_equal(one.cpu().numpy(), np.repeat(m[:1], 4, axis=0))
