"""GPU parity of the cast seam (thor_b200_cast_launch) against the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

import oracle as o
from thor_b200 import DataType, TypeConverter
from thor_b200._native import ThorB200InvalidArgument
from thor_b200.workloads import cast_input

pytestmark = pytest.mark.gpu

_TORCH_STORAGE = {o.BF16: torch.uint16, o.FP8_E4M3: torch.uint8, o.FP8_E5M2: torch.uint8}


def _to_dev(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.bool_:
        return torch.from_numpy(a.view(np.uint8).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _gpu_cast(src: np.ndarray, sdt: int, ddt: int) -> np.ndarray:
    d_src = _to_dev(src)
    n = src.size
    d_dst = torch.empty(n * np.dtype(o.STORAGE[ddt]).itemsize, dtype=torch.uint8, device="cuda")
    guard = torch.full((64,), 0xAB, dtype=torch.uint8, device="cuda")
    buf = torch.cat([d_dst, guard])  # guard bytes right behind the output: must stay untouched
    out = buf[: d_dst.numel()]
    TypeConverter.convert_type_raw(d_src.data_ptr(), out.data_ptr(), DataType(sdt), DataType(ddt), n)
    torch.cuda.synchronize()
    assert bool((buf[d_dst.numel():] == 0xAB).all()), "cast wrote past n elements"
    return out.cpu().numpy().view(o.STORAGE[ddt] if ddt != o.BOOLEAN else np.uint8)


def _assert_same(got, want, ddt):
    got = np.ascontiguousarray(got).view(np.uint8)
    want = np.ascontiguousarray(want).view(np.uint8)
    if ddt in (o.FP8_E4M3, o.FP8_E5M2):
        keep = ~np.isnan(o.to_float64(want, ddt))
        got, want = got[keep], want[keep]
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"{bad.size} byte mismatches, first at byte {bad[:5]}"


def test_configuration_1_bit_exact():
    """fp32 -> fp16, n = 2^24, U(-4,4) with +-0 / subnormal / tie / overflow edge values at 0.1 %."""
    x = cast_input(1 << 24, seed=0)
    got = _gpu_cast(x, o.FP32, o.FP16)
    want = o.cast(x, o.FP32, o.FP16)
    _assert_same(got, want, o.FP16)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 255, 2049, 65537, (1 << 20) + 3])
def test_ragged_sizes_and_no_overrun(n):
    x = cast_input(n, seed=n, edge_density=0.05)
    _assert_same(_gpu_cast(x, o.FP32, o.FP16), o.cast(x, o.FP32, o.FP16), o.FP16)
    _assert_same(_gpu_cast(x, o.FP32, o.BF16), o.cast(x, o.FP32, o.BF16), o.BF16)


def test_nan_inputs_map_to_canonical_nan():
    x = np.array([np.nan, -np.nan, 1.0, np.inf] * 5, np.float32)
    assert [int(v) for v in _gpu_cast(x, o.FP32, o.FP16).view(np.uint16)[:4]] == [0x7FFF, 0x7FFF, 0x3C00, 0x7C00]


@pytest.mark.parametrize("src", o.ALL_DTYPES, ids=lambda d: o.NAMES[d])
def test_all_pairs_on_representable_values(src):
    """Mirrors the reference's all-pairs test (TypeConverterTest.cpp:10-765): values representable in every dtype."""
    rng = np.random.default_rng(src)
    grid = rng.integers(0, 9, 4099).astype(np.float32)
    s = o.cast(grid, o.FP32, src) if src != o.FP32 else grid
    for dst in o.ALL_DTYPES:
        if dst == src:
            continue
        _assert_same(_gpu_cast(s, src, dst), o.cast(s, src, dst), dst)


@pytest.mark.parametrize("src,dst", [(o.FP32, o.FP8_E4M3), (o.FP32, o.FP8_E5M2), (o.FP64, o.FP16), (o.FP64, o.BF16), (o.FP16, o.BF16),
                                     (o.BF16, o.FP16), (o.FP16, o.FP8_E4M3), (o.BF16, o.FP8_E5M2), (o.FP64, o.FP32), (o.FP16, o.FP32),
                                     (o.FP8_E4M3, o.FP16), (o.FP8_E5M2, o.BF16), (o.INT32, o.FP16), (o.INT64, o.FP32), (o.INT64, o.BF16)])
def test_float_family_rounding(src, dst):
    rng = np.random.default_rng(7)
    base = (rng.standard_normal(1 << 16) * 2.0 ** rng.integers(-20, 18, 1 << 16)).astype(np.float64)
    if src in (o.INT32, o.INT64):
        s = (base * 1000).astype(np.int64).astype(o.STORAGE[src])
    else:
        s = o.cast(base, o.FP64, src) if src != o.FP64 else base
    _assert_same(_gpu_cast(s, src, dst), o.cast(s, src, dst), dst)


def test_float_to_int_truncates_toward_zero():
    x = np.array([-2.75, -1.5, -0.25, 0.25, 1.5, 2.75, 100.9, -100.9] * 33, np.float32)
    for dst in (o.INT8, o.INT16, o.INT32, o.INT64):
        _assert_same(_gpu_cast(x, o.FP32, dst), o.cast(x, o.FP32, dst), dst)


def test_same_dtype_and_overlap_are_rejected():
    a = torch.zeros(64, dtype=torch.float32, device="cuda")
    with pytest.raises(ThorB200InvalidArgument):
        TypeConverter.convert_type_raw(a.data_ptr(), a.data_ptr() + 256, DataType.fp32, DataType.fp32, 8)
    with pytest.raises(ThorB200InvalidArgument, match="overlap"):
        TypeConverter.convert_type_raw(a.data_ptr(), a.data_ptr() + 8, DataType.fp32, DataType.fp16, 16)


def test_in_place_same_size():
    x = np.arange(-500, 524, dtype=np.int32)
    d = torch.from_numpy(x.copy()).cuda()
    TypeConverter.convert_type_raw(d.data_ptr(), d.data_ptr(), DataType.int32, DataType.fp32, x.size)
    torch.cuda.synchronize()
    assert np.array_equal(d.cpu().numpy().view(np.float32), x.astype(np.float32))


_NP = {DataType.fp32: np.float32, DataType.fp16: np.float16, DataType.int32: np.int32, DataType.int64: np.int64, DataType.uint8: np.uint8,
       DataType.int16: np.int16, DataType.fp64: np.float64}


@pytest.mark.parametrize("src,dst", [(DataType.fp32, DataType.fp16), (DataType.fp16, DataType.fp32), (DataType.int64, DataType.uint8),
                                     (DataType.uint8, DataType.int64), (DataType.fp32, DataType.int16), (DataType.int16, DataType.fp64)])
@pytest.mark.parametrize("n", [1, 255, 8192, 8193, 20000, (1 << 20) + 77, (1 << 24)])
def test_in_place_between_element_sizes_matches_out_of_place(src, dst, n):
    """Element i of the source view becomes element i of the destination view in the same buffer
    (TypeConverterKernels.cu:846-904); compared bit for bit with the out-of-place conversion."""
    rng = np.random.default_rng(n + int(src) * 31 + int(dst))
    if src in (DataType.fp32, DataType.fp16):
        x = (rng.standard_normal(n) * 50).astype(_NP[src])
    else:
        x = rng.integers(0, 100, n).astype(_NP[src])
    ssz, dsz = x.itemsize, np.dtype(_NP[dst]).itemsize
    buf = torch.zeros(n * max(ssz, dsz) + 64, dtype=torch.uint8, device="cuda")
    buf[: n * ssz] = torch.from_numpy(x.view(np.uint8)).cuda()
    buf[n * max(ssz, dsz):] = 0xAB  # guard bytes after the larger view
    want = torch.empty(n * dsz, dtype=torch.uint8, device="cuda")
    src_copy = buf[: n * ssz].clone()
    TypeConverter.convert_type_raw(src_copy.data_ptr(), want.data_ptr(), src, dst, n)
    TypeConverter.convert_type_raw(buf.data_ptr(), buf.data_ptr(), src, dst, n)
    torch.cuda.synchronize()
    assert torch.equal(buf[: n * dsz], want)
    assert bool((buf[n * max(ssz, dsz):] == 0xAB).all())
    assert np.array_equal(want.cpu().numpy().view(_NP[dst]), o.cast(x, src, dst))


@pytest.mark.skipif(o.reference_gpu_cast_lib() is None, reason="the reference's GPU cast kernels are not built (oracle/_ref)")
@pytest.mark.parametrize("src,dst", [(o.FP32, o.FP16), (o.FP32, o.BF16), (o.FP16, o.FP32), (o.BF16, o.FP16), (o.FP32, o.FP8_E4M3), (o.FP16, o.FP8_E5M2),
                                     (o.FP32, o.INT32), (o.INT32, o.FP16), (o.UINT8, o.FP32), (o.FP32, o.BOOLEAN)])
def test_bit_identical_to_the_reference_gpu_kernels(src, dst):
    """Our kernel against TypeConverter::gpuConvertType itself (the reference's TypeConverterKernels.cu compiled
    for sm_100a), same device buffers, compared bit for bit."""
    n = (1 << 20) + 8 * 37
    if src == o.FP32:
        x = cast_input(n, seed=5)
        if dst == o.INT32:
            x = np.clip(np.nan_to_num(x, nan=0.0, posinf=1e6, neginf=-1e6), -1e6, 1e6).astype(np.float32)
        raw = x
    elif src in (o.FP16, o.BF16):
        raw = o.cast(cast_input(n, seed=6), o.FP32, src)
    elif src == o.INT32:
        raw = np.random.default_rng(7).integers(-70000, 70000, n).astype(np.int32)
    else:
        raw = np.random.default_rng(8).integers(0, 256, n).astype(np.uint8)
    pad = 64
    s_bytes, d_bytes = raw.itemsize, np.dtype(o.STORAGE[dst]).itemsize
    src_d = torch.zeros((n + pad) * s_bytes, dtype=torch.uint8, device="cuda")
    src_d[: n * s_bytes] = torch.from_numpy(raw.view(np.uint8)).cuda()
    ours = torch.zeros((n + pad) * d_bytes, dtype=torch.uint8, device="cuda")
    theirs = torch.zeros((n + pad) * d_bytes, dtype=torch.uint8, device="cuda")
    TypeConverter.convert_type_raw(src_d.data_ptr(), ours.data_ptr(), DataType(src), DataType(dst), n)
    o.reference_gpu_cast(src_d.data_ptr(), theirs.data_ptr(), src, dst, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    a, b = ours[: n * d_bytes].cpu().numpy(), theirs[: n * d_bytes].cpu().numpy()
    if dst in (o.FP16, o.BF16, o.FP32) and src in o.FLOAT_DTYPES:
        # NaN payloads are not pinned by the reference's tests: compare NaN-ness there, bits everywhere else
        av, bv = o.to_float64(a.view(o.STORAGE[dst]), dst), o.to_float64(b.view(o.STORAGE[dst]), dst)
        assert np.array_equal(np.isnan(av), np.isnan(bv))
        keep = np.repeat(~np.isnan(av), d_bytes)
        assert np.array_equal(a[keep], b[keep])
    else:
        assert np.array_equal(a, b)


def test_unaligned_views_use_the_scalar_path():
    x = cast_input(5000, seed=11)
    d = torch.from_numpy(x).cuda()
    out = torch.empty(5001, dtype=torch.float16, device="cuda")
    TypeConverter.convert_type_raw(d.data_ptr() + 4, out.data_ptr() + 2, DataType.fp32, DataType.fp16, 4999)
    torch.cuda.synchronize()
    assert np.array_equal(out[1:5000].cpu().numpy().view(np.uint16), o.cast(x[1:], o.FP32, o.FP16).view(np.uint16))


def test_in_place_resize_is_one_launch_and_matches_out_of_place_at_the_configured_size():
    """Same-address fp32 -> fp16 of 2^24 elements (and back up): one cooperative launch that walks the buffer in waves,
    instead of a chain of log(n) passes; bit-identical to the out-of-place cast."""
    import thor_b200
    from thor_b200.workloads import cast_input

    n = (1 << 24) + 3
    x = torch.from_numpy(cast_input(n, seed=3)).cuda()
    want = torch.empty(n, dtype=torch.float16, device="cuda")
    TypeConverter.convert_type(x, want)
    buf = x.clone()
    before = thor_b200.launch_count()
    TypeConverter.convert_type_raw(buf.data_ptr(), buf.data_ptr(), DataType.fp32, DataType.fp16, n)
    torch.cuda.synchronize()
    assert thor_b200.launch_count() - before == 1
    assert torch.equal(buf.view(torch.float16)[:n].view(torch.int16), want.view(torch.int16))
    # and up again, in place, from the narrow view at the start of the same buffer
    widened_want = want.float()
    before = thor_b200.launch_count()
    TypeConverter.convert_type_raw(buf.data_ptr(), buf.data_ptr(), DataType.fp16, DataType.fp32, n)
    torch.cuda.synchronize()
    assert thor_b200.launch_count() - before == 1
    assert torch.equal(buf.view(torch.int32), widened_want.view(torch.int32))


def test_copy_from_host_with_a_wider_destination_dtype_converts_in_place_on_the_gpu():
    """Tensor::copyFromAsync across placements (Tensor.cpp:769-792): fp16 host values into an fp32 device tensor travel as
    fp16 and are widened where they land; the shrinking direction is refused, as in the reference."""
    from thor_b200.type_converter import tensor_copy_from

    n = (1 << 20) + 7
    host = torch.randn(n).half().pin_memory()
    dev = torch.empty(n, dtype=torch.float32, device="cuda")
    tensor_copy_from(dev, host)
    torch.cuda.synchronize()
    assert torch.equal(dev.cpu(), host.float())
    same = torch.empty(n, dtype=torch.float16, device="cuda")
    tensor_copy_from(same, host)  # same dtype: a plain upload
    back = torch.empty(n, dtype=torch.float16).pin_memory()
    tensor_copy_from(back, same)  # and a plain download
    torch.cuda.synchronize()
    assert torch.equal(back, host)
    on_gpu = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    tensor_copy_from(on_gpu, dev)  # same GPU, different dtypes: the cast seam
    torch.cuda.synchronize()
    assert torch.equal(on_gpu, dev.bfloat16())
    with pytest.raises(Exception, match="hidden temporary"):
        tensor_copy_from(torch.empty(n, dtype=torch.float16, device="cuda"), torch.randn(n).pin_memory())
    with pytest.raises(Exception, match="CPU"):
        tensor_copy_from(torch.empty(n, dtype=torch.float32).pin_memory(), same)


def test_a_stamped_conversion_repeats_the_cast_with_one_call():
    """TypeConverter.stamp binds tensors, dtypes and stream once; run() gives what convert_type gives, and follows the
    source's current contents."""
    src = torch.randn(100_003, device="cuda")
    dst = torch.empty(100_003, device="cuda", dtype=torch.float16)
    stamped = TypeConverter.stamp(src, dst)
    want = torch.empty_like(dst)
    for _ in range(3):
        src.normal_()
        stamped.run()
        TypeConverter.convert_type(src, want)
        torch.cuda.synchronize()
        assert torch.equal(dst.view(torch.int16), want.view(torch.int16))
    with pytest.raises(Exception, match="element counts differ"):
        TypeConverter.stamp(src, dst[:5])
