"""The cases of the reference's own Python tests for this path, restated against this implementation:
same expressions, same input values, same expectations and tolerances
(bindings/python/test/core/physical/test_expression_staged_reduce.py:129-480, 827-1000, 1229-1415 and
test_expression_stable_activations.py:173-260).  The expected values are computed the way those
tests compute them: numpy in the storage dtype's compute precision, compared with rtol / atol of
1e-5 / 1e-6 (fp32), 5e-2 / 5e-2 (fp16, bf16), 1e-1 / 1e-1 (fp8 e4m3), 2e-1 / 0.5 (fp8 e5m2);
index results and stage shapes are compared exactly."""
import numpy as np
import pytest
import torch

import oracle as o
from thor_b200 import DataType
from thor_b200 import _native
from thor_b200.expression import Expression as ex

from _exprutil import from_device, to_device

pytestmark = pytest.mark.gpu

FLOAT_DTYPES = [o.FP32, o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2]
TOL = {o.FP32: (1e-5, 1e-6), o.FP16: (5e-2, 5e-2), o.BF16: (5e-2, 5e-2), o.FP8_E4M3: (1e-1, 1e-1), o.FP8_E5M2: (2e-1, 0.5)}

X3 = [[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], [[2.0, 3.0], [4.0, 5.0], [6.0, 7.0]]]
A3 = [[[4.0, 8.0], [2.0, 7.0], [5.0, 9.0]], [[6.0, 3.0], [1.0, 4.0], [8.0, 2.0]]]


def _stored(values, dtype):
    """float32 values rounded once into `dtype`: (storage array, the stored values as float64)."""
    v = np.asarray(values, dtype=np.float32)
    st = o.from_float32(v.reshape(-1), dtype).reshape(v.shape)
    return st, o.to_float64(st.reshape(-1), dtype).reshape(v.shape)


def _run(expr, inputs, dtype, **stamp_kw):
    dev = {}
    vals = {}
    for name, values in inputs.items():
        st, v64 = _stored(values, dtype)
        dev[name] = to_device(st, dtype)
        vals[name] = v64
    plan = ex.compile(expr).stamp(dev, **stamp_kw)
    plan.run()
    torch.cuda.synchronize()
    return plan, vals


def _values(plan, name="output"):
    t = plan.output(name)
    shape = tuple(t.shape)
    from thor_b200.dtypes import from_torch

    return from_device(t, int(from_torch(t.dtype))).reshape(shape)


def _close(got, want, dtype):
    rtol, atol = TOL[dtype]
    assert got.shape == tuple(np.shape(want)), (got.shape, np.shape(want))
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", [o.FP32, o.FP16, o.BF16])
def test_reduce_sum_stores_the_requested_output_dtype(dtype):
    x = ex.input("x")
    plan, v = _run(x.reduce_sum([1], squeeze_axes=[1]).with_output_dtype(DataType(dtype)), {"x": [[1.25, 2.5, 3.75], [4.0, 5.25, 6.5]]}, dtype)
    out = plan.output()
    from thor_b200.dtypes import to_torch

    assert out.dtype == to_torch(DataType(dtype)) and tuple(out.shape) == (2,)
    _close(_values(plan), v["x"].sum(axis=1), dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_reduce_sum_with_prologue_and_epilogue(dtype):
    x, y = ex.input("x"), ex.input("y")
    plan, v = _run(((x + 3.0) * (y - 1.0)).reduce_sum([1]).sqrt(), {"x": [[1.0, 2.0, 3.0, 4.0], [2.0, 3.0, 4.0, 5.0]], "y": [[1.5, 2.0, 2.5, 3.0], [1.25, 1.5, 1.75, 2.0]]},
                   dtype)
    _close(_values(plan), np.sqrt(((v["x"] + 3.0) * (v["y"] - 1.0)).sum(axis=1, keepdims=True)), dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_squeeze_rules(dtype):
    x = ex.input("x")
    keep, v = _run((x * 2.0 + 1.0).reduce_sum([1]), {"x": [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]}, dtype)
    _close(_values(keep), (v["x"] * 2.0 + 1.0).sum(axis=1, keepdims=True), dtype)  # no squeeze: reduced axes stay as 1
    both, v = _run((x + 1.0).reduce_sum([1, 2], squeeze_axes=[1, 2]), {"x": X3}, dtype)
    _close(_values(both), (v["x"] + 1.0).sum(axis=(1, 2)), dtype)
    one, v = _run(((x + 2.0) * 0.5).reduce_mean([1, 2], squeeze_axes=[2]) + 4.0, {"x": X3}, dtype)
    _close(_values(one), ((v["x"] + 2.0) * 0.5).mean(axis=(1, 2), keepdims=True).squeeze(2) + 4.0, dtype)


@pytest.mark.parametrize("dtype", [o.FP32, o.FP16, o.BF16])
def test_every_value_reduction_staged(dtype):
    x = ex.input("x")
    data = {"x": [[1.0, 2.0, 0.5], [1.5, 0.25, 4.0]]}
    cases = [
        (lambda e: (e + 0.5).reduce_prod([1]), lambda a: (a + 0.5).prod(axis=1, keepdims=True)),
        (lambda e: (e * e - 1.0).reduce_min([1]), lambda a: (a * a - 1.0).min(axis=1, keepdims=True)),
        (lambda e: (e + 1.0).reduce_max([1]) * 2.0, lambda a: (a + 1.0).max(axis=1, keepdims=True) * 2.0),
        (lambda e: (e - 1.0).reduce_norm1([1]), lambda a: np.abs(a - 1.0).sum(axis=1, keepdims=True)),
        (lambda e: (e - 1.0).reduce_norm2([1]), lambda a: np.sqrt(((a - 1.0) ** 2).sum(axis=1, keepdims=True))),
    ]
    for build, ref in cases:
        plan, v = _run(build(x), data, dtype)
        _close(_values(plan), ref(v["x"]), dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_two_reduction_boundaries(dtype):
    x, y = ex.input("x"), ex.input("y")
    first = ((x + 1.0) * y).reduce_sum([1])
    plan, v = _run((first + 2.0).reduce_mean([0], squeeze_axes=[0, 1]), {"x": [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], "y": [[0.5, 1.0, 1.5], [2.0, 2.5, 3.0]]}, dtype)
    stage1 = ((v["x"] + 1.0) * v["y"]).sum(axis=1, keepdims=True)
    _close(_values(plan), (stage1 + 2.0).mean(axis=0, keepdims=True).reshape(1), dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_reduction_chain_with_prologue_and_epilogue(dtype):
    x, y = ex.input("x"), ex.input("y")
    first = ((x + 1.0) * (y - 0.5)).reduce_sum([2])
    second = (first * 0.25 + 2.0).reduce_max([1])
    xs = [[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], [[2.0, 1.0], [4.0, 3.0], [6.0, 5.0]]]
    ys = [[[1.5, 2.0], [2.5, 3.0], [3.5, 4.0]], [[1.25, 1.75], [2.25, 2.75], [3.25, 3.75]]]
    plan, v = _run((second + 1.0).sqrt(), {"x": xs, "y": ys}, dtype)
    s1 = ((v["x"] + 1.0) * (v["y"] - 0.5)).sum(axis=2, keepdims=True)
    s2 = (s1 * 0.25 + 2.0).max(axis=1, keepdims=True)
    _close(_values(plan), np.sqrt(s2 + 1.0), dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_arg_reductions_staged(dtype):
    x, y = ex.input("x"), ex.input("y")
    ys = [[[0.0, 1.0], [3.0, 0.0], [1.0, 2.0]], [[2.0, 0.0], [0.0, 1.0], [3.0, 0.0]]]
    # several axes: the index is the row-major position inside the reduced axes
    plan, v = _run((((x + 1.0) * 0.5) - y).argmin([1, 2]), {"x": A3, "y": ys}, dtype)
    ref = ((v["x"] + 1.0) * 0.5) - v["y"]
    got = plan.output().cpu().numpy()
    assert got.dtype == np.uint32 and got.shape == (2, 1, 1)
    assert np.array_equal(got.reshape(2), ref.reshape(2, -1).argmin(axis=1).astype(np.uint32))
    # every axis
    plan, v = _run((x * 1.5 - 2.0).argmax([]), {"x": [[1.0, 5.0, 3.0], [2.0, 4.0, 6.0]]}, dtype)
    got = plan.output().cpu().numpy()
    assert got.shape == (1, 1) and int(got.reshape(-1)[0]) == int((v["x"] * 1.5 - 2.0).reshape(-1).argmax())
    # one axis, squeezed
    plan, v = _run(((x - 3.0) * (x + 1.0)).argmin([1], squeeze_axes=[1]), {"x": A3}, dtype)
    got = plan.output().cpu().numpy()
    assert np.array_equal(got, ((v["x"] - 3.0) * (v["x"] + 1.0)).argmin(axis=1).astype(np.uint32))
    # several axes, squeezed by list
    xs = [[[1.0, 9.0], [3.0, 4.0], [5.0, 2.0]], [[8.0, 0.0], [6.0, 7.0], [1.0, 3.0]]]
    plan, v = _run((x * 0.25 + 7.0).argmax([1, 2], squeeze_axes=[1, 2]), {"x": xs}, dtype)
    got = plan.output().cpu().numpy()
    assert np.array_equal(got, (v["x"] * 0.25 + 7.0).reshape(2, -1).argmax(axis=1).astype(np.uint32))


def test_arg_reductions_nan_wins_and_ties_take_the_first_index():
    x = ex.input("x")
    lo = torch.tensor([[1.0, 1.0, 3.0, 1.0], [float("nan"), 0.0, float("nan"), -4.0]], device="cuda")
    plan = ex.compile(x.argmin([1], squeeze_axes=[1])).stamp({"x": lo})
    plan.run()
    torch.cuda.synchronize()
    assert plan.output().cpu().numpy().tolist() == [0, 0]
    hi = torch.tensor([[5.0, 5.0, 3.0, 5.0], [-1.0, float("nan"), float("nan"), 8.0]], device="cuda")
    plan = ex.compile(x.argmax([1], squeeze_axes=[1])).stamp({"x": hi})
    plan.run()
    torch.cuda.synchronize()
    assert plan.output().cpu().numpy().tolist() == [0, 1]


@pytest.mark.parametrize("dtype", [o.FP32, o.FP16, o.BF16])
@pytest.mark.parametrize("is_max", [False, True])
def test_backward_of_reduce_min_and_max_with_the_default_seed(dtype, is_max):
    """No upstream gradient bound: the seed is 1, and the winner of every row receives it."""
    x = ex.input("x")
    fwd = ex.compile(x.reduce_max([1]) if is_max else x.reduce_min([1]))
    st, _ = _stored([[3.0, 1.0, 4.0], [2.0, -5.0, 0.0]], dtype)
    xd = to_device(st, dtype)
    out = torch.empty_like(xd)
    plan = fwd.compile_backward(["x"]).stamp({"x": xd}, outputs={"x_grad": out})
    assert plan.output_names() == ["x_grad"]
    plan.run()
    torch.cuda.synchronize()
    want = [[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]] if is_max else [[0.0, 1.0, 0.0], [0.0, 1.0, 0.0]]
    assert out.float().cpu().numpy().tolist() == want
    with pytest.raises((_native.ThorB200Error, _native.ThorB200InvalidArgument)):
        fwd.compile_backward(["x"]).stamp({"x": xd}, outputs={"x_grad": torch.empty(3, 2, 2, device="cuda", dtype=xd.dtype)})


def test_bf16_reductions_compute_in_fp32_not_fp16():
    st, v = _stored([[65536.0, 70000.0, 100000.0, 3.0], [1.0e6, 1.0e8, 4.0, 5.0]], o.BF16)
    plan = ex.compile((ex.input("x") + 0.0).reduce_max([1], squeeze_axes=[1])).stamp({"x": to_device(st, o.BF16)})
    plan.run()
    torch.cuda.synchronize()
    got = plan.output()
    assert got.dtype == torch.float32 and bool(torch.isfinite(got).all())
    np.testing.assert_allclose(got.cpu().numpy(), v.max(axis=1), rtol=1e-5, atol=1e-5)


EXTREME = [-1000.0, -200.0, -100.0, -80.0, -20.0, -3.0, -1.0, 0.0, 1.0, 3.0, 20.0, 80.0, 100.0, 200.0, 1000.0]


def _np_sigmoid(a):
    return np.where(a >= 0, 1.0 / (1.0 + np.exp(-np.abs(a))), np.exp(-np.abs(a)) / (1.0 + np.exp(-np.abs(a))))


@pytest.mark.parametrize("name", ["sigmoid", "softplus", "swish", "tanh", "elu", "selu", "gelu"])
def test_stable_activations_stay_finite_on_extreme_fp32_inputs(name):
    x = ex.input("x")
    a = np.array(EXTREME, dtype=np.float64)
    builders = {
        "sigmoid": (x.sigmoid(), _np_sigmoid(a)),
        "softplus": (x.softplus(), np.maximum(a, 0.0) + np.log1p(np.exp(-np.abs(a)))),
        "swish": (x.swish(), a * _np_sigmoid(a)),
        "tanh": (x.tanh(), np.tanh(a)),
        "elu": (x.elu(1.0), np.where(a > 0, a, np.expm1(np.minimum(a, 0.0)))),
        "selu": (x.selu(), 1.0507009873554805 * np.where(a > 0, a, 1.6732632423543772 * np.expm1(np.minimum(a, 0.0)))),
        "gelu": (x.gelu(), None),
    }
    expr, want = builders[name]
    plan = ex.compile(expr).stamp({"x": torch.tensor(EXTREME, device="cuda")})
    plan.run()
    torch.cuda.synchronize()
    got = plan.output().double().cpu().numpy()
    assert np.isfinite(got).all()
    if want is not None:
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_tanh_saturates_exactly():
    plan = ex.compile(ex.input("x").tanh()).stamp({"x": torch.tensor([-1000.0, -200.0, -100.0, 100.0, 200.0, 1000.0], device="cuda")})
    plan.run()
    torch.cuda.synchronize()
    assert plan.output().cpu().numpy().tolist() == [-1.0, -1.0, -1.0, 1.0, 1.0, 1.0]


def test_log1p_of_exp_keeps_the_small_term():
    vals = [-1000.0, -200.0, -100.0, -20.0, -1.0, 0.0]
    plan = ex.compile(ex.input("x").exp().log1p()).stamp({"x": torch.tensor(vals, device="cuda")})
    plan.run()
    torch.cuda.synchronize()
    got = plan.output().double().cpu().numpy()
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, np.log1p(np.exp(np.array(vals))), rtol=1e-5, atol=1e-6)
