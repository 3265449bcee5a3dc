"""The C-ABI library loads without a GPU and exports every symbol that include/thor_b200.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "thor_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"THOR_B200_API[^;(]*?\b(thor_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_symbols()
    assert "thor_b200_cast_launch" in names
    assert "thor_b200_last_error" in names


def test_library_exports_every_declared_symbol():
    import thor_b200._native as native

    for name in _declared_symbols():
        assert hasattr(native.lib, name), f"{name} declared in thor_b200.h but not exported"


def test_abi_version_and_dtype_sizes():
    import thor_b200._native as native
    from thor_b200.dtypes import SIZE, DataType

    assert native.lib.thor_b200_abi_version() == 1
    for dt in DataType:
        assert native.lib.thor_b200_dtype_size(int(dt)) == SIZE[dt]
    assert native.lib.thor_b200_dtype_size(99) == 0


def test_cast_argument_errors_need_no_gpu():
    """Same-dtype, negative-count and unknown-dtype requests are rejected before any CUDA call
    (TypeConverter.cpp:58-66 throws for equal dtypes and negative counts)."""
    import thor_b200._native as native

    with pytest.raises(native.ThorB200InvalidArgument, match="both fp32"):
        native.check(native.lib.thor_b200_cast_launch(None, None, 11, 11, 4, None))
    with pytest.raises(native.ThorB200InvalidArgument, match=">= 0"):
        native.check(native.lib.thor_b200_cast_launch(None, None, 11, 10, -1, None))
    with pytest.raises(native.ThorB200InvalidArgument, match="unknown"):
        native.check(native.lib.thor_b200_cast_launch(None, None, 11, 77, 4, None))
    # n == 0 is a no-op that needs no device
    native.check(native.lib.thor_b200_cast_launch(None, None, 11, 10, 0, None))


def test_scatter_add_descriptions_are_validated_without_a_gpu():
    """Workspace sizing of the flat scatter-add: fp32 only (as the reference, FlatScatterAddKernel.cu:236-247), four
    ping-pong arrays of num_updates 32-bit words plus the [256][tiles] digit table and the per-digit totals of four passes; the unique-and-valid policy and an
    empty update list need the one-byte placeholder only; the dependent-launch switch is a process-wide setting."""
    import thor_b200._native as native
    from thor_b200 import DataType
    from thor_b200.reductions import FlatScatterAddIndexPolicy as Policy
    from thor_b200.reductions import scatter_add_workspace_bytes as ws_bytes

    n = 100_000
    tiles = -(-n // 4096)
    align = lambda v: (v + 255) // 256 * 256
    assert ws_bytes(n, 1 << 20) == 4 * align(4 * n) + align(tiles * 256 * 4) + 4 * 256 * 4
    assert ws_bytes(n, 1 << 20, Policy.IndicesAreUniqueAndValid) == 1 and ws_bytes(0, 7) == 1
    with pytest.raises(native.ThorB200InvalidArgument, match="only fp32"):
        ws_bytes(4, 4, value_dtype=DataType.bf16)
    with pytest.raises(native.ThorB200InvalidArgument, match="2\\^31"):
        ws_bytes(1 << 31, 4)
    with pytest.raises(native.ThorB200InvalidArgument, match="2\\^32"):
        ws_bytes(4, 1 << 32)
    native.lib.thor_b200_set_dependent_launch.restype = None
    assert native.lib.thor_b200_dependent_launch() == 1
    native.lib.thor_b200_set_dependent_launch(0)
    assert native.lib.thor_b200_dependent_launch() == 0
    native.lib.thor_b200_set_dependent_launch(1)


def test_product_does_not_import_the_oracle():
    """The shipped package must never route through the CPU checker."""
    for path in list((ROOT / "thor_b200").rglob("*.py")) + list((ROOT / "thor_b200").rglob("*.cu")) + list((ROOT / "thor_b200").rglob("*.cpp")):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text and "thor_oracle" not in text, path
