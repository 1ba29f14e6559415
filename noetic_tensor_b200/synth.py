"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(no dataset is involved: the vocabulary sizes are used only as V). Generated on the device in
row chunks so that a full-size configuration never needs more than its own footprint plus one
chunk of f32 temporaries. torch is used here as a random-number source and allocator only.
"""
import math

import torch


def _chunks(rows, V, budget_elems=1 << 29):
    step = max(1, budget_elems // V)
    for r0 in range(0, rows, step):
        yield r0, min(rows, r0 + step)


def zipf_bias(V, s, gen, device):
    """log(rank^-s) over a fixed random permutation of the vocabulary: a peaked token prior."""
    perm = torch.randperm(V, generator=gen, device=device)
    rank = torch.empty(V, device=device)
    rank[perm] = torch.arange(1, V + 1, device=device, dtype=torch.float32)
    return -s * torch.log(rank)


def normal_logits(rows, V, std, dtype, gen, device, bias=None, out=None):
    out = torch.empty(rows, V, dtype=dtype, device=device) if out is None else out
    for r0, r1 in _chunks(rows, V):
        x = torch.randn(r1 - r0, V, generator=gen, device=device) * std
        if bias is not None:
            x += bias
        out[r0:r1] = x.to(dtype)
    return out


def perturbed(logits, std, gen):
    """logits + N(0, std), rounded to the logits' dtype (the frozen reference of the configs)."""
    rows, V = logits.shape
    out = torch.empty_like(logits)
    for r0, r1 in _chunks(rows, V):
        out[r0:r1] = (logits[r0:r1].float() + torch.randn(r1 - r0, V, generator=gen, device=logits.device) * std).to(logits.dtype)
    return out


def grammar_masks(rows, V, gen, device, extra=0.01, out=None):
    """U8 allow-masks: 1–4 contiguous bands of width 64–4096 per row plus `extra` random tokens."""
    out = torch.empty(rows, V, dtype=torch.uint8, device=device) if out is None else out
    col = torch.arange(V, device=device, dtype=torch.int32)[None, :]
    for r0, r1 in _chunks(rows, V, 1 << 28):
        n = r1 - r0
        m = torch.rand(n, V, generator=gen, device=device) < extra
        nb = torch.randint(1, 5, (n,), generator=gen, device=device)
        for k in range(4):
            width = torch.randint(64, 4097, (n, 1), generator=gen, device=device, dtype=torch.int32)
            start = (torch.rand(n, 1, generator=gen, device=device) * (V - 4096)).to(torch.int32)
            live = (nb > k)[:, None]
            m |= live & (col >= start) & (col < start + width)
        out[r0:r1] = m.to(torch.uint8)
    return out


def sparse_masks(rows, V, gen, device):
    """1–8 uniformly random allowed tokens per row (every tenth row exactly one); returns the
    mask and the [rows, 8] indices with −1 padding."""
    out = torch.zeros(rows, V, dtype=torch.uint8, device=device)
    k = torch.randint(1, 9, (rows,), generator=gen, device=device)
    k[::10] = 1
    idx = torch.randint(0, V, (rows, 8), generator=gen, device=device)
    live = torch.arange(8, device=device)[None, :] < k[:, None]
    r = torch.arange(rows, device=device)[:, None].expand(rows, 8)
    out[r[live], idx[live]] = 1
    return out, torch.where(live, idx, torch.full_like(idx, -1))


def uniforms(rows, gen, device):
    """One f32 uniform on [0, 1) per row with 24 random bits, the layout the sampler expects."""
    bits = torch.randint(0, 1 << 24, (rows,), generator=gen, device=device, dtype=torch.int32)
    return bits.to(torch.float32) * (1.0 / (1 << 24))


def group_relative_advantages(S, B, group, p, gen, device):
    """Bernoulli(p) rewards in groups of `group` rollouts → reward − group mean (MeanOnly), [S, B]."""
    r = (torch.rand(S, B // group, group, generator=gen, device=device) < p).to(torch.float32)
    return (r - r.mean(dim=2, keepdim=True)).reshape(S, B)


def footprint_bytes(rows, V, elem, ref, mask):
    return rows * V * (elem * (2 if ref else 1) + (1 if mask else 0))


def log2_ceil(x):
    return int(math.ceil(math.log2(max(1, x))))
