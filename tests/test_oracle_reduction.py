"""Pins the reduction / arg-reduction oracle against the hand-computed vectors of the reference's own
tests (CubReductionValueOperationsTest.cpp:23-100, 442-507; CubArgReductionTest.cpp:94-188)."""
import numpy as np

import oracle as o
from oracle import expr_oracle as eo

NAN, INF = float("nan"), float("inf")


def _t(values, shape):
    return eo.OTensor.input(np.array(values, np.float64).reshape(shape), o.FP32)


def test_value_reductions_golden():
    t = _t([-2.0, 3.0, -4.0], (3,))
    assert t.reduce_sum().v.tolist() == [-3.0] and t.reduce_prod().v.tolist() == [24.0] and t.reduce_mean().v.tolist() == [-1.0]
    assert t.reduce_min().v.tolist() == [-4.0] and t.reduce_max().v.tolist() == [3.0] and t.reduce_norm1().v.tolist() == [9.0]
    assert abs(t.reduce_norm2().v[0] - 29.0 ** 0.5) < 1e-5
    t = _t([-1.0, 2.0, -3.0, 4.0, -5.0, 6.0, -7.0, 8.0, -9.0, 10.0, -11.0, 12.0], (2, 3, 2))
    assert t.reduce_sum([1]).v.reshape(-1).tolist() == [-9.0, 12.0, -27.0, 30.0]
    assert t.reduce_prod([1]).v.reshape(-1).tolist() == [-15.0, 48.0, -693.0, 960.0]
    assert t.reduce_min([1]).v.reshape(-1).tolist() == [-5.0, 2.0, -11.0, 8.0]
    assert t.reduce_max([1]).v.reshape(-1).tolist() == [-1.0, 6.0, -7.0, 12.0]


def test_nan_propagation_and_fp16_finalisation():
    assert np.isnan(_t([1.0, NAN, -2.0], (3,)).reduce_min().v).all() and np.isnan(_t([1.0, NAN, -2.0], (3,)).reduce_max().v).all()
    m = _t([40000.0, 40000.0, -40000.0, -40000.0], (2, 2)).reduce_mean([1], out_dtype=o.FP16)
    assert m.v.reshape(-1).tolist() == [40000.0, -40000.0]
    l2 = _t([300.0, 400.0, 500.0, 1200.0], (2, 2)).reduce_norm2([1], out_dtype=o.FP16)
    assert l2.v.reshape(-1).tolist() == [500.0, 1300.0]


def test_arg_reductions_golden():
    t = _t([3.0, 1.0, 1.0, 2.0, -5.0, -1.0, -5.0, -2.0], (2, 4))
    assert t.argmin([1]).v.reshape(-1).tolist() == [1, 0] and t.argmax([1]).v.reshape(-1).tolist() == [0, 1]
    t = _t([9.0, 1.0, 5.0, 8.0, -1.0, 4.0, 0.0, 7.0, 6.0, 2.0, 3.0, -2.0], (2, 3, 2))
    assert t.argmin([1]).v.reshape(-1).tolist() == [2, 0, 0, 2] and t.argmax([1]).v.reshape(-1).tolist() == [0, 1, 1, 0]
    assert t.argmin([0, 2]).v.reshape(-1).tolist() == [2, 3, 3] and t.argmax([0, 2]).v.reshape(-1).tolist() == [0, 1, 1]
    t = _t([3.0, NAN, 2.0, NAN, 5.0, 5.0, 1.0, 1.0], (2, 4))
    assert t.argmin([1]).v.reshape(-1).tolist() == [1, 2] and t.argmax([1]).v.reshape(-1).tolist() == [1, 0]
    t = _t([INF, INF, -INF, -INF], (2, 2))
    assert t.argmin([1]).v.reshape(-1).tolist() == [0, 0] and t.argmax([1]).v.reshape(-1).tolist() == [0, 0]


def test_squeeze_rules():
    t = _t(np.arange(24), (2, 3, 4))
    assert t.reduce_sum([1]).shape == (2, 1, 4)
    assert t.reduce_sum([1], [1]).shape == (2, 4)
    assert t.reduce_sum([], [(1 << 64) - 1]).shape == (1,)
