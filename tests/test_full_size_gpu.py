"""The five benchmark configurations at their full sizes.

Where the CPU oracle finishes in seconds the whole result is compared; otherwise row-local results
are compared on a sample of rows and whole-tensor results through properties that do not depend on
the size: rows of a softmax sum to one, the position of a row's maximum survives softmax, a full
reduction equals the fold of the reductions of its shards (a checksum of checksums), column sums
are additive over row blocks."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import expr_oracle as eo
from thor_b200 import DataType, TypeConverter
from thor_b200.expression import Expression as ex
from thor_b200.workloads import cast_input

pytestmark = pytest.mark.gpu


def _bf16(t):
    return t.view(torch.uint16).cpu().numpy()


def test_c2_full_size_against_the_oracle():
    rows = cols = 8192
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(rows, cols, device="cuda", generator=g).half()
    z = torch.randn(rows, cols, device="cuda", generator=g).half()
    a = (torch.rand(cols, device="cuda", generator=g) + 0.5).half()
    e = (ex.input("a") * ex.input("x") + ex.runtime_scalar("b")).relu() * ex.input("z").sigmoid()
    plan = ex.compile(e).stamp({"a": a, "x": x, "b": 0.1, "z": z})
    plan.run()
    torch.cuda.synchronize()
    got = plan.output().cpu().numpy()
    want = o.c2_fused(a.cpu().numpy(), x.cpu().numpy(), 0.1, z.cpu().numpy(), fuse_mul_add=True)
    d = eo.ulp_distance(got.astype(np.float64), want.astype(np.float64), o.FP16)
    assert float(d.max()) <= 1.0
    assert float((got.view(np.uint16) == want.view(np.uint16)).mean()) > 0.9999


def test_c3_full_size_softmax_and_argmax():
    rows, cols = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, cols, device="cuda", generator=g) * 3.0
    xi = ex.input("x")
    ee = (xi - xi.reduce_max([1])).exp()
    y = torch.empty_like(x)
    plan = ex.compile(ee / ee.reduce_sum([1])).stamp({"x": x}, outputs={"output": y})
    arg = ex.compile(xi.argmax([1], squeeze_axes=[1])).stamp({"x": x})
    plan.run()
    arg.run()
    torch.cuda.synchronize()
    # properties over every row
    sums = y.double().sum(dim=1)
    assert float((sums - 1.0).abs().max()) <= 1e-5
    idx = arg.output().cpu().numpy()
    assert idx.dtype == np.uint32 and idx.shape == (rows,)
    assert np.array_equal(idx, torch.argmax(y, dim=1).cpu().numpy().astype(np.uint32)), "the largest probability sits where the largest logit sits"
    # the oracle on the whole tensor (about 1 GiB in, multithreaded C)
    want_y, want_idx = o.softmax_rows(x.cpu().numpy())
    assert np.array_equal(idx, want_idx)
    sample = np.random.default_rng(0).choice(rows, 512, replace=False)
    np.testing.assert_allclose(y[torch.from_numpy(sample).cuda()].cpu().numpy(), want_y[sample], rtol=1e-5, atol=1e-12)
    del want_y


def test_c3_full_size_elementwise_part_given_the_rows_own_statistics():
    """The tolerance of configuration 3 has two parts: the row statistics (fp32-accumulated, 1e-5 relative) and the
    elementwise part, at most 2 fp32 ulp GIVEN identical row statistics.  The same row program also stores its row
    maximum and row sum, so the elementwise part can be checked on its own, over all 2^28 elements on the device:
      * against the same chain in plain fp32 torch, expf(x - m) / s with the kernel's own m and s: at most 2 ulp;
      * against the ideal value exp(fl32(x - m)) / s in float64: relative error at most 2.5 * 2^-23 -- expf is
        documented at up to 2 ulp of the exponential (2 * 2^-23 relative at worst) and the IEEE division adds half an
        ulp of the quotient (2^-24 relative at worst)."""
    rows, cols = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(33)
    x = torch.randn(rows, cols, device="cuda", generator=g) * 3.0
    xi = ex.input("x")
    m_e = xi.reduce_max([1])
    ee = (xi - m_e).exp()
    s_e = ee.reduce_sum([1])
    y = torch.empty_like(x)
    plan = ex.compile({"y": ee / s_e, "s": s_e, "m": m_e}).stamp({"x": x}, outputs={"y": y})
    assert plan.physical_stage_names() == ["row_program"]
    plan.run()
    torch.cuda.synchronize()
    m, s = plan.output("m"), plan.output("s")
    assert torch.equal(m.reshape(-1), x.max(dim=1).values), "a maximum is exact"
    worst_ulp, worst_rel, worst_stat = 0, 0.0, 0.0
    for r0 in range(0, rows, 4096):
        xs, ys, ms, ss = x[r0:r0 + 4096], y[r0:r0 + 4096], m[r0:r0 + 4096].reshape(-1, 1), s[r0:r0 + 4096].reshape(-1, 1)
        same_chain = torch.exp(xs - ms) / ss  # fp32 throughout
        # both are non-negative floats: the distance in ulp is the distance of their bit patterns
        worst_ulp = max(worst_ulp, int((ys.view(torch.int32) - same_chain.view(torch.int32)).abs().max()))
        e64 = torch.exp((xs - ms).double())
        ideal = e64 / ss.double()
        normal = ideal >= 2.0 ** -126
        worst_rel = max(worst_rel, float((((ys.double() - ideal).abs() / ideal)[normal]).max()))
        worst_stat = max(worst_stat, float(((ss.double().reshape(-1) - e64.sum(dim=1)).abs() / e64.sum(dim=1)).max()))
        del same_chain, e64, ideal, normal
    assert worst_ulp <= 2, f"{worst_ulp} ulp from the fp32 chain with the same row statistics"
    assert worst_rel <= 2.5 * 2.0 ** -23, f"relative error {worst_rel / 2.0 ** -23:.2f} * 2^-23 from the ideal quotient"
    assert worst_stat <= 1e-5, f"row sums {worst_stat} relative from the float64 sums"


def test_c4_full_size_statistics_and_checksum_of_checksums():
    n = 1 << 31
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    step = 1 << 27
    for s in range(0, n, step):  # generated in blocks: an fp32 temporary of the whole vector would take 8 GiB
        x[s:s + step] = (torch.randn(step, device="cuda", generator=g) + 0.01).bfloat16()

    def build():
        xi = ex.input("x")
        return {"sum": xi.reduce_sum(), "sumsq": (xi * xi).reduce_sum(), "max": xi.reduce_max()}

    full = ex.compile(build()).stamp({"x": x})
    full.run()
    torch.cuda.synchronize()
    s_full, q_full, m_full = (float(full.output(k)) for k in ("sum", "sumsq", "max"))
    # checksum of checksums: the same program on 16 shards, folded in float64
    shards = 16
    part = ex.compile(build())
    s_acc = q_acc = 0.0
    m_acc = -np.inf
    for k in range(shards):
        p = part.stamp({"x": x[k * (n // shards):(k + 1) * (n // shards)]})
        p.run()
        torch.cuda.synchronize()
        s_acc += float(p.output("sum"))
        q_acc += float(p.output("sumsq"))
        m_acc = max(m_acc, float(p.output("max")))
    assert abs(s_full - s_acc) <= 1e-5 * abs(s_acc) + 2e-7 * n
    assert abs(q_full - q_acc) <= 1e-5 * abs(q_acc)
    assert m_full == m_acc
    # and the oracle over the whole vector (4 GiB, fp64 accumulation on the host cores)
    s, q, m = o.c4_stats(_bf16(x))
    assert abs(s_full - s) <= 1e-5 * abs(s) + 2e-7 * n
    assert abs(q_full - q) <= 1e-5 * abs(q)
    assert m_full == m


def test_c5_full_size_layernorm_forward_and_backward():
    rows, cols = 32768, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    gamma = (torch.rand(cols, device="cuda", generator=g) * 0.2 + 0.9).bfloat16()
    beta = (torch.randn(cols, device="cuda", generator=g) * 0.02).bfloat16()
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 1e-2).bfloat16()
    xe, ge, be = ex.input("x"), ex.input("gamma"), ex.input("beta")
    xc = xe - xe.reduce_mean([1])
    rstd = 1.0 / ((xc * xc).reduce_mean([1]) + 1e-5).sqrt()
    fwd_eq = ex.compile({"y": (xc * rstd * ge + be).cast(DataType.bf16)})
    fwd = fwd_eq.stamp({"x": x, "gamma": gamma, "beta": beta})
    bwd_eq = fwd_eq.compile_backward(["x", "gamma", "beta"])
    bwd = bwd_eq.stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
    fwd.run()
    bwd.run()
    torch.cuda.synchronize()
    # row-local results on a sample of rows against the oracle
    sample = torch.from_numpy(np.sort(np.random.default_rng(1).choice(rows, 256, replace=False))).cuda()
    xs, dys = x[sample].contiguous(), dy[sample].contiguous()
    want_y, _, _ = o.layernorm_fwd(_bf16(xs), _bf16(gamma), _bf16(beta), 1e-5)
    got_y = o.to_float64(_bf16(fwd.output("y")[sample].contiguous()).reshape(-1), o.BF16)
    d = eo.ulp_distance(got_y, o.to_float64(want_y.reshape(-1), o.BF16), o.BF16)
    assert float(d.max()) <= 1.0
    want_dx, _, _ = o.layernorm_bwd(_bf16(xs), _bf16(gamma), _bf16(dys), 1e-5)
    got_dx = o.to_float64(_bf16(bwd.output("x_grad")[sample].contiguous()).reshape(-1), o.BF16)
    want_dx = o.to_float64(want_dx.reshape(-1), o.BF16)
    d = eo.ulp_distance(got_dx, want_dx, o.BF16)
    d = np.where(np.abs(got_dx - want_dx) <= 2e-8, 0.0, d)  # fp32 noise of the cancelling terms, as in the small-size test
    assert float(d.max()) <= 1.0
    # column sums are additive over row blocks: full dgamma / dbeta against the fold of 8 blocks (fp64 fold)
    blocks = 8
    dg_acc = np.zeros(cols)
    db_acc = np.zeros(cols)
    for k in range(blocks):
        sl = slice(k * (rows // blocks), (k + 1) * (rows // blocks))
        p = bwd_eq.stamp({"x": x[sl], "gamma": gamma, "beta": beta, "__grad_output": dy[sl]})
        p.run()
        torch.cuda.synchronize()
        dg_acc += p.output("gamma_grad").double().cpu().numpy()
        db_acc += p.output("beta_grad").double().cpu().numpy()
    dg = bwd.output("gamma_grad").double().cpu().numpy()
    db = bwd.output("beta_grad").double().cpu().numpy()
    # every partial was rounded to bf16 once (2^-9 relative each), the full result once
    for got_c, acc in ((dg, dg_acc), (db, db_acc)):
        scale = np.abs(acc) + 1e-2 * np.sqrt(rows)
        assert float((np.abs(got_c - acc) / scale).max()) <= 2.0 ** -6
    # and the oracle for the whole column sums
    _, dg_w, db_w = o.layernorm_bwd(_bf16(x), _bf16(gamma), _bf16(dy), 1e-5)
    for got_c, want_c in ((dg, dg_w), (db, db_w)):
        dd = eo.ulp_distance(got_c, eo.round_to(want_c, o.BF16), o.BF16)
        dd = np.where(np.abs(got_c - want_c) <= 1e-5 * np.abs(want_c) + 2e-7 * rows * 1e-2 + 2.0 ** -9 * np.abs(want_c), 0.0, dd)
        assert float(dd.max()) <= 1.0


def test_c1_full_size_is_bit_exact_and_in_place_agrees():
    x = cast_input(1 << 24, seed=0)
    d = torch.from_numpy(x).cuda()
    out = torch.empty(1 << 24, dtype=torch.float16, device="cuda")
    TypeConverter.convert_type_raw(d.data_ptr(), out.data_ptr(), DataType.fp32, DataType.fp16, x.size)
    inplace = d.clone()
    TypeConverter.convert_type_raw(inplace.data_ptr(), inplace.data_ptr(), DataType.fp32, DataType.fp16, x.size)
    torch.cuda.synchronize()
    want = o.cast(x, o.FP32, o.FP16).view(np.uint16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want)
    assert np.array_equal(inplace.view(torch.float16)[: x.size].cpu().numpy().view(np.uint16), want)
