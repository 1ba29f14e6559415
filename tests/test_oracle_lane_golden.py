"""Pins of the oracle's lane operations (softmax, log_softmax, logsumexp, argmax, sum_dim) to the
reference's own tests: src/tensor/tests/standard.rs:8-24 (NaN-propagating argmax, ties),
:101-129 (logsumexp at infinities, against f64, gradient = softmax), :333-365 (backward error
bounds), src/tensor/tests/checks.rs:103-114 (NaN / all −inf rows), src/tensor/tests/ops.rs:76-78
(ties) and the operand order of src/tensor/kernels.rs:122-148."""
import math

import numpy as np

INF, NAN = float("inf"), float("nan")


def test_argmax_propagates_nan_and_takes_the_first_tie(oracle):
    v = np.array([1.0, NAN, 5.0, 2.0, NAN, 3.0, 9.0, 0.0, 4.0, NAN, NAN, 1.0, 1.0, 7.0, 7.0, 2.0], np.float32).reshape(4, 4)
    idx, val = oracle.lane_op(oracle.LANE_ARGMAX, v)
    assert idx.tolist() == [1, 0, 1, 1]
    assert np.isnan(val[:3]).all() and val[3] == 7.0
    ties = np.array([1.0, 3.0, 3.0, 2.0, 5.0, 5.0, 5.0, 0.0], np.float32).reshape(2, 4)
    assert oracle.lane_op(oracle.LANE_ARGMAX, ties)[0].tolist() == [1, 0]


def test_logsumexp_at_infinities_and_against_f64(oracle):
    v = np.array([1000.0, 1000.0, -INF, 0.0, -INF, -INF, -INF, -INF, 1.0, INF, 0.0, 2.0, 0.5, NAN, 1.0, 3.0], np.float32).reshape(4, 4)
    out = oracle.lane_op(oracle.LANE_LOGSUMEXP, v)
    assert np.float32(out[0]) == np.float32(1000.0) + np.float32(math.log(2.0)), "no overflow"
    assert out[1] == -INF and out[2] == INF and np.isnan(out[3])
    x = np.random.default_rng(41).uniform(-30, 30, (3, 50)).astype(np.float32)
    y, g = oracle.lane_op(oracle.LANE_LOGSUMEXP, x, upstream=np.ones(3))
    xd = x.astype(np.float64)
    m = xd.max(axis=1)
    want = m + np.log(np.exp(xd - m[:, None]).sum(axis=1))
    assert (np.abs(y - want) <= 4 * np.finfo(np.float32).eps * np.maximum(np.abs(want), 1.0)).all()
    assert np.abs(g - oracle.lane_op(oracle.LANE_SOFTMAX, x)).max() <= 1e-6, "its gradient is the softmax"
    d = oracle.lane_op(oracle.LANE_LOGSUMEXP, np.array([[0.1, 0.2, 0.3]]), dtype=oracle.F64)
    assert abs(d[0] - math.log(math.exp(0.1) + math.exp(0.2) + math.exp(0.3))) < 1e-15


def test_softmax_of_nan_and_fully_masked_rows(oracle):
    v = np.array([0.5, NAN, -1.0, 2.0, -INF, -INF, -INF, -INF, 1.0, -INF, 3.0, -INF], np.float32).reshape(3, 4)
    for op in (oracle.LANE_SOFTMAX, oracle.LANE_LOG_SOFTMAX):
        y = oracle.lane_op(op, v)
        assert np.isnan(y[:2]).all(), "a NaN or all-(−inf) row gives NaN"
        assert not np.isnan(y[2]).any()
    y = oracle.lane_op(oracle.LANE_SOFTMAX, v)[2]
    assert y[1] == 0.0 and y[3] == 0.0 and abs(y[0] + y[2] - 1.0) < 1e-7


def test_softmax_backward_errors_stay_within_the_reference_bounds(oracle):
    for length, rows, sm_bound, lsm_bound in ((17, 600, 7.9e-5, 1.3e-6), (1000, 100, 3.0e-6, 9.1e-7)):
        g = np.random.default_rng(97)
        x = g.uniform(-6, 6, (rows, length)).astype(np.float32)
        w = g.uniform(-1, 1, (rows, length)).astype(np.float32)
        xd, wd = x.astype(np.float64), w.astype(np.float64)
        e = np.exp(xd - xd.max(axis=1, keepdims=True))
        p = e / e.sum(axis=1, keepdims=True)
        for op, bound, want in ((oracle.LANE_SOFTMAX, sm_bound, p * (wd - (wd * p).sum(axis=1, keepdims=True))),
                                (oracle.LANE_LOG_SOFTMAX, lsm_bound, wd - p * wd.sum(axis=1, keepdims=True))):
            _, got = oracle.lane_op(op, x, upstream=wd)
            worst = (np.abs(got - want) / np.abs(want).max(axis=1, keepdims=True)).max()
            assert worst <= bound, (op, length, worst)


def test_sum_dim_is_the_eight_partial_order(oracle):
    g = np.random.default_rng(3)
    for V in (1, 7, 8, 9, 64, 1001):
        x = g.normal(0, 100, (5, V)).astype(np.float32)
        want = []
        for row in x:
            p = [np.float32(0)] * 8
            full = V // 8
            for j in range(full):
                for k in range(8):
                    p[k] = np.float32(p[k] + row[8 * j + k])
            acc = np.float32(0)
            for k in range(4):
                acc = np.float32(acc + np.float32(p[k] + p[k + 4]))
            for e in row[8 * full:]:
                acc = np.float32(acc + e)
            want.append(acc)
        got = oracle.lane_op(oracle.LANE_SUM, x).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), np.array(want, np.float32).view(np.uint32)), V
