"""Sharding the path across the GPUs of one box: rows are independent, so each rank takes a
contiguous range of sequences and no data crosses between GPUs. Only a `TokenReduction` that
spans ranks (Sum, TokenMean, SequenceMean per seed) needs the ranks' per-sequence partial sums,
which are gathered once (two floats per sequence) and folded in sequence order by the library's
own kernels — so the value has the bits of the one-GPU `nrl_reduce_tokens` whatever the number
of ranks.

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


def gather_sequences(local, S, B, group=None):
    """All ranks' per-sequence rows ([n_seq, k] each), concatenated in rank order = sequence
    order, on every rank: the one collective of the path (a few bytes per sequence)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    ranges = [sequence_range(S, B, r, world) for r in range(world)]
    width = max(e - b for b, e in ranges)
    padded = torch.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded.contiguous(), group=group)
    return torch.cat([out[r][: e - b] for r, (b, e) in enumerate(ranges)]).contiguous()


class ShardedReduction:
    """`TokenReduction` (src/nn/rl.rs:69-92) of per-token values whose sequences are spread over
    the ranks: `per` and `mask` are this rank's [n_seq, T] slices (sequences
    `sequence_range(S, B, rank, world)`), `per` already zero at unscored positions.

    All arithmetic is libnrl's: `nrl_reduce_tokens_partial` sums each local sequence to a pair
    (one warp per sequence), the pairs are gathered in sequence order, `nrl_reduce_tokens_fold`
    folds each seed's pairs — the two steps `nrl_reduce_tokens` runs in one kernel, so `value` has
    the bits of the one-GPU call for any number of ranks. `backward(g_out)` gives this rank's
    d_per [n_seq, T] from the gradient of the whole reduced value, the divisors taken from the
    gathered counts (`nrl_reduce_tokens_bwd_pairs`).

    `kernels` replaces the three library calls (partial, fold, backward): the CPU test of the
    gather plumbing passes host stand-ins with the kernels' operand order; product code never does."""

    def __init__(self, per, mask, reduction, S, B, group=None, kernels=None):
        if reduction == NONE:
            raise ValueError("TokenReduction::None is local: nothing to combine")
        if kernels is None:
            from . import ops

            kernels = (ops.reduce_tokens_partial, ops.reduce_tokens_fold, ops.reduce_tokens_backward_pairs)
        partial, fold, self._bwd = kernels
        self.reduction, self.S, self.B, self.T = reduction, S, B, per.shape[1]
        self.mask, self.n_seq = mask, per.shape[0]
        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        rank = dist.get_rank(group) if world > 1 else 0
        self.seq_begin, seq_end = sequence_range(S, B, rank, world)
        if per.shape[0] != seq_end - self.seq_begin:
            raise ValueError(f"this rank holds sequences [{self.seq_begin}, {seq_end}) of {S * B}, got {per.shape[0]}")
        self.pairs = gather_sequences(partial(per, mask), S, B, group)
        self.value = fold(self.pairs, S, B, reduction)

    def backward(self, g_out):
        return self._bwd(self.reduction, self.S, self.B, self.T, self.seq_begin, self.n_seq, self.pairs, self.mask, g_out.contiguous())


def reduce_tokens_sharded(per, mask, reduction, S, B, group=None, kernels=None):
    """The reduced tensor alone: [S] (Sum, TokenMean, SequenceMean) or [S, B] (PerSequence), on every rank."""
    return ShardedReduction(per, mask, reduction, S, B, group, kernels).value
