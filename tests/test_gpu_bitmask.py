"""Bit-packed vocabulary masks read by the row kernels themselves (NRL_FWD_MASK_BITS /
nrl_row_bwd_args.mask_bits): every kernel the byte-mask path can take — grouped, one block per
row, split rows, the element-wise loop for ragged V, temperature — must give bit-identical
results to the same call with the byte mask, forward and backward."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def pack_bits(m):
    rows, V = m.shape
    pad = (-V) % 32
    b = np.packbits(np.pad(m != 0, ((0, 0), (0, pad))), axis=1, bitorder="little")
    return torch.from_numpy(b.view(np.int32).reshape(rows, -1).copy())


def same(a, b, what):
    if a is None and b is None:
        return
    va = a.view(torch.int32) if a.dtype == torch.float32 else a
    vb = b.view(torch.int32) if b.dtype == torch.float32 else b
    assert torch.equal(va, vb), what


CASES = [  # rows, V, dtype, ref, temperature, mask density
    (1400, 128256, torch.bfloat16, True, 1.0, "grammar"),   # grouped kernel
    (1400, 32000, torch.float32, False, 1.0, 0.3),          # grouped kernel, f32
    (400, 128256, torch.bfloat16, True, 1.0, "grammar"),    # one block per row
    (9, 151936, torch.bfloat16, True, 1.0, 0.02),           # split rows
    (33, 1001, torch.float32, True, 1.0, 0.5),              # ragged V: element-wise loop
    (29, 4104, torch.bfloat16, True, 0.7, 0.4),             # temperature: the general path
    (64, 262144, torch.bfloat16, True, 1.0, "sparse"),      # 1-8 allowed tokens per row
    (17, 40, torch.float32, False, 1.0, 0.6),
]


@pytest.mark.parametrize("rows,V,dtype,ref,tau,density", CASES)
def test_bit_masks_equal_byte_masks(rows, V, dtype, ref, tau, density):
    from noetic_tensor_b200 import ops, synth

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(rows + V)
    x = synth.normal_logits(rows, V, 3.0, dtype, gen, dev)
    r = synth.perturbed(x, 0.05, gen) if ref else None
    if density == "grammar":
        m = synth.grammar_masks(rows, V, gen, dev)
    elif density == "sparse":
        m = synth.sparse_masks(rows, V, gen, dev)
    else:
        m = (torch.rand(rows, V, generator=gen, device=dev) < density).to(torch.uint8)
        m[:, 0] = 1
    if isinstance(m, tuple):
        m = m[0]
    bits = pack_bits(m.cpu().numpy()).to(dev)
    u = synth.uniforms(rows, gen, dev)
    for mode in ("sample", "greedy", "stats"):
        kw = dict(uniforms=u) if mode == "sample" else (dict(greedy=True) if mode == "greedy" else {})
        a = ops.row_forward(x, ref_logits=r, allow=m, temperature=tau, **kw)
        b = ops.row_forward(x, ref_logits=r, allow_bits=bits, temperature=tau, **kw)
        for name in ("tokens", "logp", "ref_logp", "kl", "entropy", "rowstats", "status"):
            same(getattr(a, name), getattr(b, name), (mode, name))
    # given tokens (the log-prob of one element per row: the single-element mask read), allowed and excluded ones
    f = ops.row_forward(x, ref_logits=r, allow=m, temperature=tau, uniforms=u)
    given = f.tokens.clone()
    given[::3] = torch.randint(0, V, (given[::3].numel(),), generator=gen, device=dev, dtype=torch.int32)
    a = ops.row_forward(x, ref_logits=r, allow=m, temperature=tau, tokens=given)
    b = ops.row_forward(x, ref_logits=r, allow_bits=bits, temperature=tau, tokens=given)
    for name in ("logp", "ref_logp", "kl", "entropy", "status"):
        same(getattr(a, name), getattr(b, name), ("given tokens", name))
    score = (torch.rand(rows, generator=gen, device=dev) < 0.8).float()
    kw = dict(g_logp=score, g_ent=-0.01 * score, temperature=tau)
    if ref:
        kw["g_kl"] = 0.04 * score
    da = ops.row_backward(x, f, ref_logits=r, allow=m, **kw)
    db = ops.row_backward(x, f, ref_logits=r, allow_bits=bits, **kw)
    same(da, db, "d(logits)")
    # one mask row broadcast to all rows
    a = ops.row_forward(x, ref_logits=r, allow=m[:1].contiguous(), temperature=tau, uniforms=u)
    b = ops.row_forward(x, ref_logits=r, allow_bits=bits[:1].contiguous(), temperature=tau, uniforms=u)
    same(a.tokens, b.tokens, "broadcast tokens")
    same(a.logp, b.logp, "broadcast logp")


def test_bit_mask_argument_checks():
    from noetic_tensor_b200 import ops

    dev = torch.device("cuda:0")
    x = torch.zeros(4, 64, device=dev)
    u = torch.full((4,), 0.5, device=dev)
    with pytest.raises(ValueError):
        ops.row_forward(x, allow_bits=torch.zeros(4, 1, dtype=torch.int32, device=dev), uniforms=u)  # 64 tokens need 2 words
    none = ops.row_forward(x, allow_bits=torch.zeros(4, 2, dtype=torch.int32, device=dev), uniforms=u)
    assert none.status.cpu().tolist() == [1, 1, 1, 1] and none.tokens.cpu().tolist() == [-1] * 4
    bits = torch.tensor([[1 << 5, 0]] * 4, dtype=torch.int32, device=dev)
    one = ops.row_forward(x, allow_bits=bits, uniforms=u)
    assert one.tokens.cpu().tolist() == [5] * 4 and (one.logp.abs() < 1e-6).all()
