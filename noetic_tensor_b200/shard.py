"""Sharding the path across the GPUs of one box: rows are independent, so each rank takes a
contiguous range of sequences and no data crosses between GPUs. Only a `TokenReduction` that
spans ranks (Sum, TokenMean, SequenceMean per seed) needs the ranks' per-sequence partial sums,
which are gathered once (a few floats per sequence) and folded in sequence order — so the value
is bitwise the same whatever the number of ranks.

The reference has no counterpart on this path: its multi-device story is gradient data parallel
over TCP (src/nn/dist), with one process per device (src/tensor/cuda/backend.rs:106-109), which
is the process model kept here.
"""
import torch
import torch.distributed as dist

NONE, SUM, TOKEN_MEAN, PER_SEQUENCE, SEQUENCE_MEAN = range(5)


def sequence_range(S, B, rank, world):
    """Sequences [begin, end) of the flattened [S·B] axis owned by `rank`: the split falls on
    sequence boundaries, seeds first (S), then sequences within a seed (B)."""
    n = S * B
    return n * rank // world, n * (rank + 1) // world


def row_range(S, B, T, rank, world):
    b, e = sequence_range(S, B, rank, world)
    return b * T, e * T


def local_sequence_partials(per, mask):
    """Per-sequence sums and scored counts of this rank's [n_seq, T] per-token values (already
    zero at unscored positions). Sums run over T in index order in f64."""
    sums = per.to(torch.float64).sum(dim=1)
    counts = (mask if mask is not None else torch.ones_like(per)).to(torch.float64).sum(dim=1)
    return sums, counts


def gather_sequences(local, S, B, group=None):
    """All ranks' per-sequence values, concatenated in rank order = sequence order, on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    width = max(sequence_range(S, B, r, world)[1] - sequence_range(S, B, r, world)[0] for r in range(world))
    padded = torch.zeros(width, dtype=local.dtype, device=local.device)
    padded[: local.numel()] = local
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    pieces = []
    for r in range(world):
        b, e = sequence_range(S, B, r, world)
        pieces.append(out[r][: e - b])
    return torch.cat(pieces)


def reduce_tokens_sharded(per, mask, reduction, S, B, group=None):
    """`TokenReduction` (src/nn/rl.rs:69-92) of per-token values sharded by sequence: `per` and
    `mask` are this rank's [n_seq, T] slices. Returns the full reduced tensor on every rank:
    [S] (Sum, TokenMean, SequenceMean) or [S, B] (PerSequence)."""
    if reduction == NONE:
        raise ValueError("TokenReduction::None is local: nothing to combine")
    sums, counts = local_sequence_partials(per, mask)
    sums = gather_sequences(sums, S, B, group).reshape(S, B)
    counts = gather_sequences(counts, S, B, group).reshape(S, B)
    per_seq = sums / counts.clamp_min(1.0)
    if reduction == PER_SEQUENCE:
        return per_seq.to(torch.float32)
    out = torch.zeros(S, dtype=torch.float64, device=sums.device)
    for b in range(B):  # fold in sequence order: the same additions whatever the number of ranks
        if reduction == SUM or reduction == TOKEN_MEAN:
            out = out + sums[:, b]
        else:
            out = out + per_seq[:, b]
    if reduction == TOKEN_MEAN:
        out = out / counts.sum(dim=1).clamp_min(1.0)
    if reduction == SEQUENCE_MEAN:
        out = out / (counts > 0).to(torch.float64).sum(dim=1).clamp_min(1.0)
    return out.to(torch.float32)
