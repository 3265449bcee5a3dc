"""Leading-dimension sharding across the GPUs of one box and the one collective the path needs.

Elementwise stages, casts, row reductions and row programs need no communication: every rank runs
the same kernels on its own contiguous block of rows.  Only values reduced over the sharded
dimension (full reductions, LayerNorm dgamma / dbeta column sums) are combined, with one allreduce
of the per-rank fp32 partials.  The reference has no multi-GPU path; this is new glue over
``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, rank: int, world: int, multiple: int = 8) -> Tuple[int, int]:
    """Contiguous [start, stop) of `n` rows / elements for `rank`; every boundary but the last is a
    multiple of `multiple` (16-byte packs stay aligned), sizes differ by at most `multiple`."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    blocks = -(-n // multiple)
    per, extra = divmod(blocks, world)
    start_block = rank * per + min(rank, extra)
    stop_block = start_block + per + (1 if rank < extra else 0)
    return min(n, start_block * multiple), min(n, stop_block * multiple)


def ordered_keys(values: torch.Tensor, nan_wins_high: bool) -> torch.Tensor:
    """int32 keys whose signed order is the float order of `values` (fp32), with every NaN mapped to the key that wins a
    maximum (nan_wins_high) or a minimum.  The reduction seam's rule -- a NaN in any shard is the result -- survives an
    integer max / min across ranks, which the backends' floating-point max / min do not promise."""
    bits = values.contiguous().view(torch.int32)
    keys = torch.where(bits >= 0, bits, bits ^ 0x7FFFFFFF)
    nan_key = 0x7FFFFFFF if nan_wins_high else -0x80000000
    return torch.where(torch.isnan(values), torch.full_like(keys, nan_key), keys)


def from_ordered_keys(keys: torch.Tensor) -> torch.Tensor:
    """Inverse of ordered_keys (the winning NaN keys are NaN bit patterns themselves)."""
    return torch.where(keys >= 0, keys, keys ^ 0x7FFFFFFF).view(torch.float32)


def combine_partials(sums: Optional[torch.Tensor] = None, maxima: Optional[torch.Tensor] = None, minima: Optional[torch.Tensor] = None,
                     group=None) -> None:
    """In-place allreduce of per-rank fp32 partials: `sums` with SUM (sum, sum of squares, dgamma, dbeta ...),
    `maxima` with MAX, `minima` with MIN; extremes are NaN-propagating like the single-GPU reductions (they cross the
    ranks as ordered integer keys).  No-op without an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    if sums is not None:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
    if maxima is not None:
        keys = ordered_keys(maxima, True)
        dist.all_reduce(keys, op=dist.ReduceOp.MAX, group=group)
        maxima.copy_(from_ordered_keys(keys).reshape(maxima.shape))
    if minima is not None:
        keys = ordered_keys(minima, False)
        dist.all_reduce(keys, op=dist.ReduceOp.MIN, group=group)
        minima.copy_(from_ordered_keys(keys).reshape(minima.shape))


def finalize_mean(total: torch.Tensor, global_count: int) -> torch.Tensor:
    """Mean of a sharded reduction: divide the allreduced fp32 sum by the global element count (fp32 division,
    like the reduction seam's finaliser)."""
    return total / torch.tensor(float(global_count), dtype=torch.float32, device=total.device)


class Communicator:
    """The C ABI's NCCL allreduce (thor_b200_comm_*), for callers that do not go through torch.distributed.
    Rank 0 creates the id with ``Communicator.unique_id()`` and hands the 128 bytes to the other ranks."""

    def __init__(self, nranks: int, rank: int, unique_id: bytes):
        import ctypes as C

        from . import _native

        self._lib = _native.lib
        self._lib.thor_b200_comm_init.argtypes = [C.c_int, C.c_int, C.c_char_p, C.POINTER(C.c_void_p)]
        self._lib.thor_b200_comm_allreduce_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
        self._lib.thor_b200_comm_allreduce_stats_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p]
        self._lib.thor_b200_comm_destroy.argtypes = [C.c_void_p]
        self._lib.thor_b200_comm_destroy.restype = None
        if len(unique_id) != 128:
            raise ValueError("the NCCL id is 128 bytes")
        self._h = C.c_void_p()
        _native.check(self._lib.thor_b200_comm_init(nranks, rank, unique_id, C.byref(self._h)))

    @staticmethod
    def unique_id() -> bytes:
        import ctypes as C

        from . import _native

        buf = C.create_string_buffer(128)
        _native.lib.thor_b200_comm_unique_id.argtypes = [C.c_char_p]
        _native.check(_native.lib.thor_b200_comm_unique_id(buf))
        return buf.raw

    def allreduce(self, t: torch.Tensor, op: str = "sum", stream=None) -> None:
        from . import _native

        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("allreduce takes a contiguous fp32 CUDA tensor")
        _native.check(self._lib.thor_b200_comm_allreduce_f32(self._h, t.data_ptr(), t.numel(), {"sum": 0, "max": 1, "min": 2}[op], _native.stream_handle(stream)))

    def allreduce_stats(self, sums: Optional[torch.Tensor] = None, maxima: Optional[torch.Tensor] = None, minima: Optional[torch.Tensor] = None,
                        stream=None) -> None:
        """One NCCL group for the statistics of a sharded reduction step: `sums` added, `maxima` / `minima` combined with
        NaN-propagating max / min, all in place (thor_b200_comm_allreduce_stats_f32)."""
        from . import _native

        args = []
        for t in (sums, maxima, minima):
            if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
                raise ValueError("allreduce_stats takes contiguous fp32 CUDA tensors")
            args += [t.data_ptr() if t is not None else None, t.numel() if t is not None else 0]
        _native.check(self._lib.thor_b200_comm_allreduce_stats_f32(self._h, *args, _native.stream_handle(stream)))

    def close(self) -> None:
        if self._h:
            self._lib.thor_b200_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BoundCombinerSlot:
    """One slot of a Combiner bound to its buffers: wait() and submit() are single C calls."""

    def __init__(self, combiner, slot, sums, maxima, minima, rounded_sums, stream):
        import ctypes as C

        from . import _native
        from .dtypes import from_torch

        def pair(t):
            if t is None:
                return C.c_void_p(None), C.c_uint64(0)
            if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
                raise ValueError("partials are contiguous fp32 CUDA tensors")
            return C.c_void_p(t.data_ptr()), C.c_uint64(t.numel())

        if rounded_sums is not None and (sums is None or rounded_sums.numel() != sums.numel() or not rounded_sums.is_contiguous()):
            raise ValueError("rounded_sums must be contiguous and hold as many elements as sums")
        self._keep = (combiner, sums, maxima, minima, rounded_sums)
        st = _native.stream_handle(stream)
        self._check = _native.check
        self._wait, self._wait_args = combiner._lib.thor_b200_combiner_wait, (combiner._h, slot, st)
        self._submit = combiner._lib.thor_b200_combiner_submit
        self._submit_args = (combiner._h, slot, st, *pair(sums), *pair(maxima), *pair(minima),
                             C.c_void_p(rounded_sums.data_ptr()) if rounded_sums is not None else C.c_void_p(None),
                             int(from_torch(rounded_sums.dtype)) if rounded_sums is not None else 0)

    def wait(self) -> None:
        status = self._wait(*self._wait_args)
        if status:
            self._check(status)

    def submit(self) -> None:
        status = self._submit(*self._submit_args)
        if status:
            self._check(status)


class Combiner:
    """Overlapped combine of a stepping job's partials (thor_b200_combiner_*): the statistics of step i cross the ranks on
    the combiner's own high-priority stream while the kernel of step i + 1 runs.  The caller keeps `slots` copies of its
    partial buffers and uses slot i % slots in step i: wait(slot) before the step's kernels, submit(slot, ...) after them."""

    def __init__(self, comm: Communicator, slots: int = 2):
        import ctypes as C

        from . import _native

        self._lib = _native.lib
        L = self._lib
        L.thor_b200_combiner_create.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]
        L.thor_b200_combiner_wait.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.thor_b200_combiner_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int]
        L.thor_b200_combiner_drain.argtypes = [C.c_void_p, C.c_void_p]
        L.thor_b200_combiner_stream.argtypes = [C.c_void_p]
        L.thor_b200_combiner_stream.restype = C.c_void_p
        L.thor_b200_combiner_destroy.argtypes = [C.c_void_p]
        L.thor_b200_combiner_destroy.restype = None
        self._comm = comm  # keeps the communicator alive
        self._h = C.c_void_p()
        _native.check(L.thor_b200_combiner_create(comm._h, slots, C.byref(self._h)))
        self.stream = torch.cuda.ExternalStream(L.thor_b200_combiner_stream(self._h))

    def wait(self, slot: int, stream=None) -> None:
        from . import _native

        _native.check(self._lib.thor_b200_combiner_wait(self._h, slot, _native.stream_handle(stream)))

    def submit(self, slot: int, sums: Optional[torch.Tensor] = None, maxima: Optional[torch.Tensor] = None, minima: Optional[torch.Tensor] = None,
               rounded_sums: Optional[torch.Tensor] = None, stream=None) -> None:
        """Combine behind everything `stream` (default: the current stream) holds so far; rounded_sums, when given, receives
        the combined sums converted to its dtype."""
        from . import _native
        from .dtypes import from_torch

        def pair(t):
            if t is None:
                return None, 0
            if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
                raise ValueError("partials are contiguous fp32 CUDA tensors")
            return t.data_ptr(), t.numel()

        if rounded_sums is not None and (sums is None or rounded_sums.numel() != sums.numel() or not rounded_sums.is_contiguous()):
            raise ValueError("rounded_sums must be contiguous and hold as many elements as sums")
        _native.check(self._lib.thor_b200_combiner_submit(self._h, slot, _native.stream_handle(stream), *pair(sums), *pair(maxima), *pair(minima),
                                                          rounded_sums.data_ptr() if rounded_sums is not None else None,
                                                          int(from_torch(rounded_sums.dtype)) if rounded_sums is not None else 0))

    def drain(self, stream=None) -> None:
        from . import _native

        _native.check(self._lib.thor_b200_combiner_drain(self._h, _native.stream_handle(stream)))

    def bind(self, slot: int, sums: Optional[torch.Tensor] = None, maxima: Optional[torch.Tensor] = None, minima: Optional[torch.Tensor] = None,
             rounded_sums: Optional[torch.Tensor] = None, stream=None) -> "BoundCombinerSlot":
        """wait / submit of one slot with its buffers and stream (the current one when none is given) resolved once, for
        stepping loops in which the Python side of a call would cost as much as the step."""
        return BoundCombinerSlot(self, slot, sums, maxima, minima, rounded_sums, stream)

    def close(self) -> None:
        if self._h:
            self._lib.thor_b200_combiner_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
