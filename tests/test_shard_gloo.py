"""The multi-rank path on CPU: two gloo ranks each own a range of sequences, exchange only their
per-sequence partial sums, and must produce the single-rank `TokenReduction` values to the bit
(and the reference's values within its f32 tolerance)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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


def _rank_main(rank, world, port, S, B, T, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from noetic_tensor_b200 import shard

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    per, mask = _case(S, B, T)
    b, e = shard.sequence_range(S, B, rank, world)
    lp = torch.from_numpy(per.reshape(S * B, T)[b:e].copy())
    lm = torch.from_numpy(mask.reshape(S * B, T)[b:e].copy())
    res = {r: shard.reduce_tokens_sharded(lp, lm, r, S, B).numpy() for r in (shard.SUM, shard.TOKEN_MEAN, shard.PER_SEQUENCE, shard.SEQUENCE_MEAN)}
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **{str(k): v for k, v in res.items()})
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
    single = {r: shard.reduce_tokens_sharded(torch.from_numpy(per.reshape(S * B, T)), torch.from_numpy(mask.reshape(S * B, T)), r, S, B).numpy()
              for r in (shard.SUM, shard.TOKEN_MEAN, shard.PER_SEQUENCE, shard.SEQUENCE_MEAN)}
    mp.spawn(_rank_main, args=(2, _free_port(), S, B, T, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        got = np.load(tmp_path / f"rank{rank}.npz")
        for r, want in single.items():
            assert np.array_equal(got[str(r)].view(np.int32), want.view(np.int32)), (rank, r)
    # and the values are the reference's reductions (CpuRef f32) of the same per-token values:
    # policy_gradient_loss with logp = −per and unit weights gives per-token values `per`
    for r, want in single.items():
        ref = oracle.rl_eval(oracle.OP_PG, (S, B, T, 1), dtype=oracle.F32, logp=-per.astype(np.float64), weights=np.ones((S, B, T)), mask=mask.astype(np.float64), reduction=r)
        assert np.max(np.abs(want.ravel() - ref) / (1 + np.abs(ref))) <= 1e-5, r
