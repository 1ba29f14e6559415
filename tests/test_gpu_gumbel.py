"""The reference's own sampler on the device (nrl_sample_gumbel): Gumbel-max with one ChaCha20
u64 per logit must give the tokens the CPU restatement of `sample_categorical`
(src/nn/rl.rs:490-529) gives for the same seed and stream position — all of them, not only off
some boundary: the noise is regenerated from the same counter-based stream."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

INF = float("inf")


def dev():
    return torch.device("cuda:0")


def stored(x, dtype):
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dev()).to(dtype)
    host = t.view(torch.int16).cpu().numpy().view(np.uint16) if dtype == torch.bfloat16 else t.cpu().numpy()
    return t, host


@pytest.mark.parametrize("rows,V,dtype", [(64, 16, torch.float32), (40, 1000, torch.bfloat16), (12, 4104, torch.float32), (6, 32000, torch.bfloat16), (33, 37, torch.bfloat16), (5, 1001, torch.float32)])
@pytest.mark.parametrize("tau", [1.0, 0.7])
def test_tokens_are_the_reference_samplers(oracle, rows, V, dtype, tau):
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(rows * V)
    x, xh = stored(g.uniform(-3, 3, (rows, V)), dtype)
    seed = oracle.derive_seed(5, "sampler test")
    want = oracle.sample_gumbel(xh, tau, 5, "sampler test")
    tok, status = ops.sample_gumbel(x, seed, temperature=tau)
    assert (status == 0).all()
    assert np.array_equal(tok.cpu().numpy().astype(np.int64), want)
    # entering the stream later: the rows from r0 on, 2·r0·V words in
    r0 = rows // 3
    tok2, _ = ops.sample_gumbel(x[r0:].contiguous(), seed, word_offset=2 * r0 * V, temperature=tau)
    assert np.array_equal(tok2.cpu().numpy().astype(np.int64), want[r0:])
    # the same call again: identical
    assert torch.equal(tok, ops.sample_gumbel(x, seed, temperature=tau)[0])


def test_masks_and_refusals(oracle):
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(7)
    rows, V = 48, 96
    x, xh = stored(g.uniform(-3, 3, (rows, V)), torch.float32)
    seed = oracle.derive_seed(11, "device sampler")
    # every seventh token excluded, as the reference's device test does (src/nn/tests/gpu/rl.rs:157-174)
    for fill in (-INF, -1e9):
        add = np.where(np.arange(V) % 7 == 3, fill, 0.0).astype(np.float32)[None]
        want = oracle.sample_gumbel(xh, 0.7, 11, "device sampler", add_mask=add)
        tok, status = ops.sample_gumbel(x, seed, temperature=0.7, add_mask=torch.from_numpy(add).to(dev()))
        assert (status == 0).all() and np.array_equal(tok.cpu().numpy().astype(np.int64), want)
        assert (tok.cpu().numpy() % 7 != 3).all()
    allow = (g.uniform(0, 1, (rows, V)) < 0.3).astype(np.uint8)
    allow[:, 5] = 1
    want = oracle.sample_gumbel(xh, 1.0, 11, "device sampler", allow=allow)
    tok, status = ops.sample_gumbel(x, seed, allow=torch.from_numpy(allow).to(dev()))
    assert (status == 0).all() and np.array_equal(tok.cpu().numpy().astype(np.int64), want)
    # a row with no allowed token, and a NaN: refused with the status bits of the row forward
    allow[3] = 0
    x2 = x.clone()
    x2[9, 4] = float("nan")
    tok, status = ops.sample_gumbel(x2, seed, allow=torch.from_numpy(allow).to(dev()))
    assert status[3] == 1 and tok[3] == -1 and status[9] == 2 and tok[9] == -1
    ok = np.ones(rows, bool)
    ok[[3, 9]] = False
    assert np.array_equal(tok.cpu().numpy().astype(np.int64)[ok], want[ok]), "the other rows draw from their own stream positions"
    with pytest.raises(RuntimeError, match="no allowed token"):
        oracle.sample_gumbel(x2.cpu().numpy(), 1.0, 11, "device sampler", allow=allow)


def test_frequencies_match_the_distribution(oracle):
    # src/nn/tests/rl.rs:582-629: 40 000 draws within 4.5 standard errors, the excluded token never
    from noetic_tensor_b200 import ops

    draws = 40_000
    row = np.array([0.4, -1.0, 1.2, 3.0, 0.0, -0.3], dtype=np.float32)
    mrow = np.array([[0.0, 0.0, 0.0, -INF, 0.5, 0.0]], dtype=np.float32)
    x = torch.from_numpy(np.tile(row, (draws, 1))).to(dev())
    tok, status = ops.sample_gumbel(x, oracle.derive_seed(5, "sampler test"), temperature=0.7, add_mask=torch.from_numpy(mrow).to(dev()))
    z = row.astype(np.float64) / np.float32(0.7) + mrow[0]
    p = np.exp(z - z.max())
    p /= p.sum()
    fr = np.bincount(tok.cpu().numpy(), minlength=6) / draws
    assert fr[3] == 0 and np.all(np.abs(fr - p) <= 4.5 * np.sqrt(p * (1 - p) / draws) + 1e-12)
    want = oracle.sample_gumbel(np.tile(row, (draws, 1)), 0.7, 5, "sampler test", add_mask=mrow)
    assert np.array_equal(tok.cpu().numpy().astype(np.int64), want)


def test_full_vocabulary_rows_at_speed(oracle):
    """V = 128256 bf16: the device tokens equal the CPU sampler's on every row of a sample, and the
    kernel's rate is printed (it is arithmetic-bound: a ChaCha20 block and 16 f64 logs per 8 logits)."""
    from noetic_tensor_b200 import ops, synth

    gen = torch.Generator(device=dev())
    gen.manual_seed(3)
    rows, V = 2048, 128256
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev())
    m = synth.grammar_masks(rows, V, gen, dev())
    seed = oracle.derive_seed(2, "bench")
    tok, status = ops.sample_gumbel(x, seed, allow=m)
    assert (status == 0).all() and m[torch.arange(rows, device=dev()), tok.long()].all()
    n = 12
    xh = x[:n].view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.sample_gumbel(xh, 1.0, 2, "bench", allow=m[:n].cpu().numpy())
    assert np.array_equal(tok[:n].cpu().numpy().astype(np.int64), want)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        ops.sample_gumbel(x, seed, allow=m)
    e1.record()
    torch.cuda.synchronize()
    print(f"device Gumbel-max sampler: {rows * 3 / (e0.elapsed_time(e1) * 1e-3) / 1e3:.1f} K rows/s at V = {V}")
