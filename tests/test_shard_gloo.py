"""The multi-rank path on CPU: two gloo ranks each own a range of sequences, exchange only their
per-sequence pairs, and must produce the single-rank `TokenReduction` values to the bit (and the
reference's values within its f32 tolerance), forward and backward. There is no GPU here, so the
three library kernels are replaced by host stand-ins with the kernels' operand order
(tests/truth.py); tests/test_gpu_losses.py holds the kernels themselves to those stand-ins' bits
on a GPU, and bench.py runs the same gather over NCCL."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _host_kernels():
    import truth

    t = torch.from_numpy
    return (lambda per, mask: t(truth.warp_seq_pairs(per.numpy(), None if mask is None else mask.numpy())),
            lambda pairs, S, B, r: t(truth.fold_pairs(pairs.numpy(), S, B, r)),
            lambda r, S, B, T, b, n, pairs, mask, g: t(truth.bwd_pairs(r, S, B, T, b, n, pairs.numpy(), None if mask is None else mask.numpy(), g.numpy())))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(S=3, B=5, T=7, seed=0):
    g = np.random.default_rng(seed)
    mask = (g.uniform(0, 1, (S, B, T)) < 0.7).astype(np.float32)
    mask[0, 0] = 0.0  # a sequence with no scored position
    per = (g.normal(0, 2, (S, B, T)).astype(np.float32)) * mask
    return per, mask


def _upstream(S, B, r):
    g = np.random.default_rng(100 + r)
    return g.normal(0, 1, (S, B) if r == 3 else (S,)).astype(np.float32)


def _rank_main(rank, world, port, S, B, T, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist

    from noetic_tensor_b200 import shard

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    per, mask = _case(S, B, T)
    b, e = shard.sequence_range(S, B, rank, world)
    lp = torch.from_numpy(per.reshape(S * B, T)[b:e].copy())
    lm = torch.from_numpy(mask.reshape(S * B, T)[b:e].copy())
    res = {}
    for r in (shard.SUM, shard.TOKEN_MEAN, shard.PER_SEQUENCE, shard.SEQUENCE_MEAN):
        red = shard.ShardedReduction(lp, lm, r, S, B, kernels=_host_kernels())
        res[str(r)] = red.value.numpy()
        res[f"d{r}"] = red.backward(torch.from_numpy(_upstream(S, B, r))).numpy()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **res)
    dist.destroy_process_group()


def test_partition_covers_every_sequence_once():
    from noetic_tensor_b200 import shard

    for S, B, world in ((8, 32, 8), (4, 256, 8), (3, 5, 2), (1, 1, 4)):
        seen = []
        for r in range(world):
            b, e = shard.sequence_range(S, B, r, world)
            seen += list(range(b, e))
        assert seen == list(range(S * B))
    assert shard.row_range(8, 32, 1024, 3, 8) == (3 * 32 * 1024, 4 * 32 * 1024)


@pytest.mark.timeout(120)
def test_two_gloo_ranks_match_one_rank_bitwise(tmp_path, oracle):
    from noetic_tensor_b200 import shard

    S, B, T = 3, 5, 7
    per, mask = _case(S, B, T)
    reds = (shard.SUM, shard.TOKEN_MEAN, shard.PER_SEQUENCE, shard.SEQUENCE_MEAN)
    one = {r: shard.ShardedReduction(torch.from_numpy(per.reshape(S * B, T)), torch.from_numpy(mask.reshape(S * B, T)), r, S, B, kernels=_host_kernels()) for r in reds}
    single = {r: one[r].value.numpy() for r in reds}
    single_d = {r: one[r].backward(torch.from_numpy(_upstream(S, B, r))).numpy() for r in reds}
    mp.spawn(_rank_main, args=(2, _free_port(), S, B, T, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        got = np.load(tmp_path / f"rank{rank}.npz")
        b, e = shard.sequence_range(S, B, rank, 2)
        for r, want in single.items():
            assert np.array_equal(got[str(r)].view(np.int32), want.view(np.int32)), (rank, r)
            assert np.array_equal(got[f"d{r}"].view(np.int32), single_d[r][b:e].view(np.int32)), (rank, r, "backward")
    # and the values and gradients are the reference's (CpuRef f32) for the same per-token values:
    # policy_gradient_loss with logp = −per and unit weights gives per-token values `per`, d loss / d logp = −d_per
    for r, want in single.items():
        ref, gref = oracle.rl_eval(oracle.OP_PG, (S, B, T, 1), dtype=oracle.F32, logp=-per.astype(np.float64), weights=np.ones((S, B, T)), mask=mask.astype(np.float64), reduction=r,
                                   upstream=_upstream(S, B, r).astype(np.float64))
        assert np.max(np.abs(want.ravel() - ref) / (1 + np.abs(ref))) <= 1e-5, r
        assert np.max(np.abs(-single_d[r].ravel() - gref) / (1 + np.abs(gref))) <= 1e-5, (r, "backward")
