"""GPU parity of the generic lane operations (nrl_lane_op) against the CPU oracle's restatement of
the reference engine: softmax, log_softmax, logsumexp with their backward rules, the
NaN-propagating first-maximum argmax and the lane sum in the reference's operand order.
Tolerances: values and gradients within 1e-5 relative or 1e-6 absolute of the f64 oracle;
argmax indices equal; the lane sum bit-equal to Cpu(Reference) for f32 input."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

INF, NAN = float("inf"), float("nan")
SHAPES = [(5, 1), (7, 3), (9, 8), (33, 17), (21, 256), (13, 1001), (6, 4104), (3, 32000), (2, 128256)]


def dev():
    return torch.device("cuda:0")


def put(x, dtype):
    """(device tensor in `dtype`, the values it stores as float32 numpy)."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dev()).to(dtype).contiguous()
    return t, t.float().cpu().numpy()


def close(got, want, what, rel=1e-5, ab=1e-6):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, what
    both_nan = np.isnan(got) & np.isnan(want)
    same_inf = np.isinf(want) & (got == want)
    ok = both_nan | same_inf | (np.abs(got - want) <= ab) | (np.abs(got - want) <= rel * np.abs(want))
    assert ok.all(), f"{what}: worst |Δ| {np.nanmax(np.abs(got - want)[~(both_nan | same_inf)]):.3e}"


@pytest.mark.parametrize("rows,V", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_values(oracle, rows, V, dtype):
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(rows * 1000 + V)
    xt, xh = put(g.normal(0, 3, (rows, V)), dtype)
    close(ops.softmax(xt).cpu().numpy(), oracle.lane_op(oracle.LANE_SOFTMAX, xh, dtype=oracle.F64), "softmax")
    close(ops.log_softmax(xt).cpu().numpy(), oracle.lane_op(oracle.LANE_LOG_SOFTMAX, xh, dtype=oracle.F64), "log_softmax")
    close(ops.logsumexp(xt).cpu().numpy(), oracle.lane_op(oracle.LANE_LOGSUMEXP, xh, dtype=oracle.F64), "logsumexp")
    idx, val = ops.argmax(xt)
    oi, ov = oracle.lane_op(oracle.LANE_ARGMAX, xh)
    assert np.array_equal(idx.cpu().numpy().astype(np.int64), oi) and np.array_equal(val.cpu().numpy(), ov.astype(np.float32))
    got = ops.sum_last(xt).cpu().numpy()
    want = oracle.lane_op(oracle.LANE_SUM, xh).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "the lane sum is bit-equal to Cpu(Reference)"
    again = ops.softmax(xt)
    assert torch.equal(again.view(torch.int32), ops.softmax(xt).view(torch.int32)), "bitwise run to run"


@pytest.mark.parametrize("rows,V", SHAPES)
def test_backward_rules(oracle, rows, V):
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(rows * 77 + V)
    xt, xh = put(g.normal(0, 2, (rows, V)), torch.float32)
    up = g.uniform(-1, 1, (rows, V)).astype(np.float32)
    upt = torch.from_numpy(up).to(dev())
    for fwd, bwd, op in ((ops.softmax, ops.softmax_backward, oracle.LANE_SOFTMAX), (ops.log_softmax, ops.log_softmax_backward, oracle.LANE_LOG_SOFTMAX)):
        y = fwd(xt)
        _, want = oracle.lane_op(op, xh, dtype=oracle.F64, upstream=up.astype(np.float64))
        got = bwd(y, upt).cpu().numpy()
        scale = np.abs(want).max(axis=1, keepdims=True) + 1e-30
        assert (np.abs(got - want) / scale).max() <= 2e-5, f"backward of op {op}: {(np.abs(got - want) / scale).max():.2e} of the row's largest gradient"
    ur = g.uniform(-1, 1, rows).astype(np.float32)
    lse = ops.logsumexp(xt)
    _, want = oracle.lane_op(oracle.LANE_LOGSUMEXP, xh, dtype=oracle.F64, upstream=ur.astype(np.float64))
    got = ops.logsumexp_backward(xt, lse, torch.from_numpy(ur).to(dev())).cpu().numpy()
    close(got, want, "logsumexp backward", rel=2e-5, ab=1e-6)


def test_infinities_nan_and_ties(oracle):
    """The reference's edge cases: src/tensor/tests/standard.rs:8-24, 101-109, checks.rs:103-114."""
    from noetic_tensor_b200 import ops

    v = np.array([1000.0, 1000.0, -INF, 0.0, -INF, -INF, -INF, -INF, 1.0, INF, 0.0, 2.0, 0.5, NAN, 1.0, 3.0], np.float32).reshape(4, 4)
    out = ops.logsumexp(torch.from_numpy(v).to(dev())).cpu().numpy()
    assert abs(out[0] - (1000.0 + np.log(2.0))) <= 1e-4 and out[1] == -INF and out[2] == INF and np.isnan(out[3])
    a = np.array([1.0, NAN, 5.0, 2.0, NAN, 3.0, 9.0, 0.0, 4.0, NAN, NAN, 1.0, 1.0, 7.0, 7.0, 2.0], np.float32).reshape(4, 4)
    idx, val = ops.argmax(torch.from_numpy(a).to(dev()))
    assert idx.cpu().tolist() == [1, 0, 1, 1] and np.isnan(val.cpu().numpy()[:3]).all() and val.cpu().numpy()[3] == 7.0
    ties = np.array([1.0, 3.0, 3.0, 2.0, 5.0, 5.0, 5.0, 0.0, -INF, -INF, -INF, -INF], np.float32).reshape(3, 4)
    assert ops.argmax(torch.from_numpy(ties).to(dev()))[0].cpu().tolist() == [1, 0, 0]
    s = np.array([0.5, NAN, -1.0, 2.0, -INF, -INF, -INF, -INF, 1.0, -INF, 3.0, -INF], np.float32).reshape(3, 4)
    for f, op in ((ops.softmax, oracle.LANE_SOFTMAX), (ops.log_softmax, oracle.LANE_LOG_SOFTMAX)):
        y = f(torch.from_numpy(s).to(dev())).cpu().numpy()
        assert np.isnan(y[:2]).all() and not np.isnan(y[2]).any()
        close(y, oracle.lane_op(op, s), "edge rows")
    # the same edge rows inside long lanes that take the 16-byte path, a NaN late in the row
    big = np.random.default_rng(1).normal(0, 1, (4, 4096)).astype(np.float32)
    big[0, 4000] = NAN
    big[1] = -INF
    big[2, 17] = INF
    bt = torch.from_numpy(big).to(dev())
    close(ops.logsumexp(bt).cpu().numpy(), oracle.lane_op(oracle.LANE_LOGSUMEXP, big), "logsumexp, long edge rows")
    close(ops.softmax(bt).cpu().numpy(), oracle.lane_op(oracle.LANE_SOFTMAX, big), "softmax, long edge rows")
    oi, _ = oracle.lane_op(oracle.LANE_ARGMAX, big)
    assert np.array_equal(ops.argmax(bt)[0].cpu().numpy().astype(np.int64), oi)


@pytest.mark.parametrize("V,dtype", [(32000, torch.float32), (50264, torch.float32), (128256, torch.float32), (151936, torch.float32), (65536, torch.bfloat16), (128256, torch.bfloat16), (262144, torch.bfloat16)])
def test_long_rows_held_by_a_cluster(oracle, V, dtype):
    """softmax / log_softmax of rows too long for L2 to keep (a thread-block cluster of 2 to 8 CTAs
    holds the row in shared memory): values against the f64 oracle, the reference's edge rows (a NaN
    late in the row, a row of −inf, a +inf, −inf runs as long as a CTA's slice), more rows than
    resident clusters, and the same bits run to run."""
    from noetic_tensor_b200 import ops

    g = np.random.default_rng(V)
    rows = 70
    x = g.normal(0, 3, (rows, V)).astype(np.float32)
    x[0, V - 5] = NAN
    x[1] = -INF
    x[2, 17] = INF
    x[3, : V // 2] = -INF          # whole slices without a finite value
    x[4, V // 3:] = -INF
    x[5, 1:] = -INF                 # a single finite value
    x[6] = 1e30                     # exp(0) everywhere
    xt, xh = put(x, dtype)
    for f, op in ((ops.softmax, oracle.LANE_SOFTMAX), (ops.log_softmax, oracle.LANE_LOG_SOFTMAX)):
        y = f(xt)
        got = y.cpu().numpy()
        close(got[:8], oracle.lane_op(op, xh[:8], dtype=oracle.F64), "edge rows")
        idx = g.choice(np.arange(8, rows), 4, replace=False)
        close(got[idx], oracle.lane_op(op, xh[idx], dtype=oracle.F64), "values")
        assert np.isnan(got[0]).all() and np.isnan(got[1]).all() and np.isnan(got[2]).all()
        assert torch.equal(f(xt).view(torch.int32), y.view(torch.int32)), "bitwise run to run"
    s = ops.softmax(xt)[8:].double().sum(dim=1)
    assert ((s - 1).abs() < 1e-4).all()


def test_many_rows_and_throughput():
    """More rows than resident blocks (the grid-stride loop), checked through properties, and the
    rate of each op at the Llama-3 vocabulary printed for the record."""
    from noetic_tensor_b200 import ops

    gen = torch.Generator(device=dev())
    gen.manual_seed(2)
    rows, V = 4096, 128256
    x = torch.randn(rows, V, generator=gen, device=dev(), dtype=torch.float32) * 3
    y = ops.softmax(x)
    assert ((y.sum(dim=1) - 1).abs() < 1e-4).all() and (y >= 0).all()
    ly = ops.log_softmax(x)
    assert (ly.exp() - y).abs().max() < 1e-6
    lse = ops.logsumexp(x)
    assert (torch.logsumexp(x, dim=1) - lse).abs().max() < 1e-4
    idx, val = ops.argmax(x)
    tv, ti = x.max(dim=1)
    assert torch.equal(idx.long(), ti) and torch.equal(val, tv)
    assert (ops.sum_last(x) - x.double().sum(dim=1).float()).abs().max() < 0.5
    g = torch.randn(rows, V, generator=gen, device=dev(), dtype=torch.float32)
    dx = ops.log_softmax_backward(ly, g)
    assert dx.sum(dim=1).abs().max() < 0.5
    for name, f, nbytes in (("softmax", lambda: ops.softmax(x), 8), ("log_softmax", lambda: ops.log_softmax(x), 8), ("logsumexp", lambda: ops.logsumexp(x), 4),
                            ("argmax", lambda: ops.argmax(x), 4), ("sum_last (reference order)", lambda: ops.sum_last(x), 4),
                            ("log_softmax backward", lambda: ops.log_softmax_backward(ly, g), 12), ("softmax backward", lambda: ops.softmax_backward(y, g), 12)):
        for _ in range(3):
            f()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            f()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 5
        print(f"lane op {name}: {rows / ms / 1e3:.2f} M rows/s at V={V} f32, {rows * V * nbytes / ms / 1e6:.0f} GB/s of algorithmic bytes")
