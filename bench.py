#!/usr/bin/env python
"""Benchmark of the hot path: fused expression / reduction / cast kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2] [--no-extras]

A step is one pass of the hot path over one batch of synthetic input resident in HBM.  The headline
workload is configuration 2 (y = relu(a*x + b) * sigmoid(z), fp16 [8192, 8192], a per column, b an
fp32 runtime scalar); with N > 1 every rank owns its own [8192, 8192] row shard of a [8192*N, 8192]
problem (weak scaling, no data-path collective).  The other configurations are timed the same way
and reported under "all_configs" (their full-reduction / dgamma partials are combined with one NCCL
allreduce when N > 1).

Timing: W >= 3 warm-up steps, then exactly K steps between a barrier + synchronize on both sides,
bracketed by CUDA events on the launching stream; the max over ranks is reported.  Buffers rotate
over several disjoint sets whose total size is several times the 126 MB L2, so no step finds its
inputs in cache.  SM clocks and throttle reasons are sampled with nvidia-smi during the timed region.

Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
ROW_PROGRAM = None  # --row-program: layout fields of the row programs (A/B runs of one kernel shape against another)
FALLBACK_HBM_GBS = 6650.0


# ---------------------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------------------
def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def sample_count(self) -> int:
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in Path(self.path).read_text().strip().splitlines() if r.strip()]
            os.unlink(self.path)
        except Exception:
            rows = []
        clocks, reasons = [], set()
        for r in rows:
            try:
                clocks.append(float(r[0]))
                out["sm_max_mhz"] = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        if clocks:
            clocks.sort()
            # median of the upper half: the samples taken while the kernels were running
            busy = clocks[len(clocks) // 2:]
            out["sm_mhz"] = busy[len(busy) // 2]
        out["reasons"] = sorted(reasons)
        out["samples"] = len(clocks)
        return out


class Dist:
    def __init__(self, n_gpus: int):
        import torch

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.enabled = self.world > 1
        torch.cuda.set_device(self.local_rank if self.enabled else 0)
        if self.enabled:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        import torch

        if self.enabled:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max(self, v: float) -> float:
        import torch

        if not self.enabled:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_reduce(self, t, op="sum"):
        if self.enabled:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM if op == "sum" else self.dist.ReduceOp.MAX)

    def close(self):
        if self.enabled:
            self.dist.destroy_process_group()


def time_steps(dist: Dist, step, steps: int, warmup: int, sampler: ClockSampler | None = None, sample: bool = False, drain=None):
    """W untimed + K timed calls of step(i); returns (device ms per step as max over ranks, wall ms per step).
    `drain` (optional) makes the timing stream wait for work the steps put on side streams, so that it ends inside the
    timed region."""
    import torch

    for i in range(warmup):
        step(i)
    dist.barrier()
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        step(warmup + i)
    if drain is not None:
        drain()
    e1.record()
    dist.barrier()
    wall = (time.perf_counter() - t0) * 1e3 / steps
    ms = dist.max(e0.elapsed_time(e1) / steps)
    clocks = None
    if sample:
        # nvidia-smi cannot sample faster than every ~20 ms: when the timed region was shorter than 400 ms every rank
        # keeps the identical load running (untimed; the count derives from the rank-maximum time, so all ranks agree
        # and collectives stay matched) until a handful of samples under load exist
        extended = 0
        if steps * ms < 400.0:
            extended = int(400.0 / max(ms, 1e-3)) + 1
            for i in range(extended):
                step(warmup + steps + i)
            dist.barrier()
        if sampler:
            clocks = sampler.stop()
            clocks["untimed_extension_steps"] = extended
    return ms, wall, clocks


# ---------------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    description = ""
    dtype = ""
    unit_name = "elements"

    def __init__(self, dist: Dist, scale: float = 1.0):
        self.dist = dist
        self.scale = scale  # fraction of the leading dimension (profiling captures use a smaller case)
        self.sets = []
        self.launches_per_step = 0
        for attr in ("ROWS", "N"):
            if hasattr(self, attr) and scale != 1.0:
                setattr(self, attr, max(8, int(getattr(type(self), attr) * scale) // 8 * 8))

    def algorithmic_bytes(self) -> int: raise NotImplementedError
    def units(self) -> int: raise NotImplementedError
    def setup(self): raise NotImplementedError
    def step(self, i: int): raise NotImplementedError
    def n_sets(self, bytes_per_set: int) -> int:
        return max(2, min(8, -(-4 * L2_BYTES // max(1, bytes_per_set))))


class C1Cast(Workload):
    name = "c1_cast_fp32_fp16"
    description = "TypeConverter fp32->fp16, 1-D, n=2^24, U(-4,4) with edge values at 0.1% (per GPU)"
    dtype = "f32->f16"
    N = 1 << 24

    def setup(self):
        import torch

        from thor_b200 import TypeConverter
        from thor_b200.workloads import cast_input

        self.n = self.N
        host = torch.from_numpy(cast_input(self.n, seed=self.dist.rank))
        k = self.n_sets(self.algorithmic_bytes())
        self.sets = [(host.cuda(), torch.empty(self.n, dtype=torch.float16, device="cuda")) for _ in range(k)]
        self.convert = TypeConverter.convert_type
        self.launches_per_step = 1
        self.host_in = host.pin_memory()
        self.host_out = torch.empty(self.n, dtype=torch.float16).pin_memory()

    def algorithmic_bytes(self): return self.N * 6
    def units(self): return self.N
    def step(self, i):
        src, dst = self.sets[i % len(self.sets)]
        self.convert(src, dst)

    def e2e_step(self, i):
        src, dst = self.sets[i % len(self.sets)]
        src.copy_(self.host_in, non_blocking=True)
        self.convert(src, dst)
        self.host_out.copy_(dst, non_blocking=True)

    def e2e_bytes(self): return self.N * 4, self.N * 2


class C1CastReferenceGpu(C1Cast):
    """Baseline, not product: the reference's own TypeConverterKernels.cu, compiled unmodified for sm_100a into
    oracle/_ref, on the same buffers and timing protocol as C1 (only listed when that build is present)."""
    is_baseline = True
    name = "c1_cast_fp32_fp16_reference_gpu_kernels"
    description = "the reference's TypeConverter::gpuConvertType fp32->fp16, n=2^24 (baseline beside c1)"

    def setup(self):
        import torch

        import oracle
        from thor_b200.workloads import cast_input

        if oracle.reference_gpu_cast_lib() is None:
            raise RuntimeError("oracle/_ref/libthor_ref_gpu_cast.so is not built")
        self.n = self.N
        host = torch.from_numpy(cast_input(self.n, seed=self.dist.rank))
        k = self.n_sets(self.algorithmic_bytes())
        pad = 64  # the reference's kernels may read a few elements past n (it pads every tensor)
        self.sets = []
        for _ in range(k):
            src = torch.zeros(self.n + pad, dtype=torch.float32, device="cuda")
            src[: self.n] = host.cuda()
            self.sets.append((src, torch.empty(self.n + pad, dtype=torch.float16, device="cuda")))
        stream = torch.cuda.current_stream().cuda_stream
        self.convert = lambda s, d: oracle.reference_gpu_cast(s.data_ptr(), d.data_ptr(), oracle.FP32, oracle.FP16, self.n, stream)
        self.launches_per_step = 1
        self.kernel_kind = ["reference convertOutOfPlaceKernel"]


class C2FusedExpr(Workload):
    name = "c2_fused_relu_axb_sigmoid"
    description = "y = relu(a*x + b) * sigmoid(z): x,z,y fp16 [8192,8192] per GPU, a fp16 [8192] per column, b fp32 runtime scalar 0.1"
    dtype = "f16"
    ROWS, COLS = 8192, 8192

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(1234 + self.dist.rank)
        self.a = torch.empty(C, device="cuda", dtype=torch.float32).uniform_(0.5, 1.5, generator=gen).half()
        eq = ex.compile(((ex.input("a") * ex.input("x") + ex.runtime_scalar("b")).max(0.0)) * ex.input("z").sigmoid())
        self.eq = eq
        k = self.n_sets(self.algorithmic_bytes())
        self.sets = []
        for _ in range(k):
            x = torch.randn(R, C, device="cuda", dtype=torch.float32, generator=gen).half()
            z = torch.randn(R, C, device="cuda", dtype=torch.float32, generator=gen).half()
            y = torch.empty(R, C, device="cuda", dtype=torch.float16)
            plan = eq.stamp({"a": self.a, "x": x, "z": z, "b": 0.1}, outputs={"output": y})
            self.sets.append((plan, x, z, y))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()
        self.host_x = self.sets[0][1].cpu().pin_memory()
        self.host_z = self.sets[0][2].cpu().pin_memory()
        self.host_y = torch.empty(R, C, dtype=torch.float16).pin_memory()

    def algorithmic_bytes(self): return 3 * self.ROWS * self.COLS * 2 + self.COLS * 2
    def units(self): return self.ROWS * self.COLS
    def step(self, i): self.sets[i % len(self.sets)][0].run()

    E2E_CHUNKS = 16

    def _e2e_setup(self):
        """End to end through the public API on host buffers: the rows are cut into chunks, each with its own stamped plan,
        and upload, kernel and download of consecutive chunks run on three streams, so the two directions of the host link
        work at the same time.  Everything is ordered after the caller's stream at the start of a step and the caller's
        stream waits for all three at the end, so events on the caller's stream bracket the whole step."""
        import torch

        plan0, x, z, y = self.sets[0]
        self.e2e_streams = [torch.cuda.Stream() for _ in range(3)]
        self.e2e_chunks = []
        rows = self.ROWS
        n = min(self.E2E_CHUNKS, rows)
        for c in range(n):
            r0, r1 = rows * c // n, rows * (c + 1) // n
            plan = self.eq.stamp({"a": self.a, "x": x[r0:r1], "z": z[r0:r1], "b": 0.1}, outputs={"output": y[r0:r1]})
            self.e2e_chunks.append((plan, r0, r1, torch.cuda.Event(), torch.cuda.Event()))
        self.e2e_done = [torch.cuda.Event() for _ in range(3)]

    def e2e_step(self, i):
        import torch

        if not hasattr(self, "e2e_chunks"):
            self._e2e_setup()
        _, x, z, y = self.sets[0]
        up, run, down = self.e2e_streams
        cur = torch.cuda.current_stream()
        for st in self.e2e_streams:
            st.wait_stream(cur)
        for plan, r0, r1, uploaded, computed in self.e2e_chunks:
            with torch.cuda.stream(up):
                x[r0:r1].copy_(self.host_x[r0:r1], non_blocking=True)
                z[r0:r1].copy_(self.host_z[r0:r1], non_blocking=True)
                uploaded.record(up)
            run.wait_event(uploaded)
            plan.run(run)
            computed.record(run)
            down.wait_event(computed)
            with torch.cuda.stream(down):
                self.host_y[r0:r1].copy_(y[r0:r1], non_blocking=True)
        for st in self.e2e_streams:
            cur.wait_stream(st)

    def e2e_bytes(self): return 2 * self.ROWS * self.COLS * 2, self.ROWS * self.COLS * 2

    # CPU baseline: the oracle's C port of the same per-node-fp16 arithmetic on a row sample
    def cpu_sample(self, rows: int, threads: int):
        import numpy as np

        import oracle

        x = self.host_x[:rows].numpy()
        z = self.host_z[:rows].numpy()
        a = self.a.cpu().numpy()
        t0 = time.perf_counter()
        oracle.c2_fused(a, x, 0.1, z, True, threads)
        dt = time.perf_counter() - t0
        return (3 * rows * self.COLS * 2 + self.COLS * 2) / dt / 1e9, f"{rows} of {self.ROWS} rows x {self.COLS} cols, one pass"


class C2ReferenceGpu(C2FusedExpr):
    """Baseline, not product: the kernel that the reference's own CudaSourceEmitter::emitSpecializedBroadcast generates
    for configuration 2 (built from the reference checkout into oracle/_ref, compiled with NVRTC and the reference's
    flags, launched with its geometry: one half2 per thread, 131072 CTAs), on the same buffers and timing protocol."""
    is_baseline = True
    name = "c2_fused_relu_axb_sigmoid_reference_gpu_kernel"
    description = "the reference's emitted specialized-broadcast kernel for configuration 2 (baseline beside c2)"

    def setup(self):
        import torch

        import oracle
        from oracle.refkernel import ReferenceBroadcastKernel

        if oracle.reference_emitter_lib() is None:
            raise RuntimeError("oracle/_ref/libthor_ref_emit.so is not built")
        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(1234 + self.dist.rank)
        self.a = torch.empty(C, device="cuda", dtype=torch.float32).uniform_(0.5, 1.5, generator=gen).half()
        self.ref = ReferenceBroadcastKernel("in:a in:x mul rs:b add lit:0 max in:z sigmoid mul", {"a": oracle.FP16, "x": oracle.FP16, "b": oracle.FP32, "z": oracle.FP16},
                                            {"a": (C,), "x": (R, C), "z": (R, C)})
        self.sets = []
        for _ in range(self.n_sets(self.algorithmic_bytes())):
            x = torch.randn(R, C, device="cuda", dtype=torch.float32, generator=gen).half()
            z = torch.randn(R, C, device="cuda", dtype=torch.float32, generator=gen).half()
            self.sets.append((None, x, z, torch.empty(R, C, device="cuda", dtype=torch.float16)))
        self.launches_per_step = 1
        self.kernel_kind = ["reference specialized broadcast (half2 per thread)"]

    def step(self, i):
        _, x, z, y = self.sets[i % len(self.sets)]
        self.ref.launch({"a": self.a, "x": x, "b": 0.1, "z": z}, y)


class C3Softmax(Workload):
    name = "c3_softmax_rows_fp32"
    description = "exp(x - max_row) / sum_row(exp(x - max_row)) on fp32 [65536,4096] per GPU (composed expression)"
    dtype = "f32"
    ROWS, COLS = 65536, 4096

    def build(self, ex):
        x = ex.input("x")
        e = (x - x.reduce_max([1])).exp()
        return {"y": e / e.reduce_sum([1])}

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(77 + self.dist.rank)
        eq = ex.compile(self.build(ex))
        self.sets = []
        for _ in range(2):
            x = torch.randn(R, C, device="cuda", generator=gen) * 3.0
            y = torch.empty(R, C, device="cuda")
            self.sets.append((eq.stamp({"x": x}, outputs={"y": y}), x, y))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()

    def algorithmic_bytes(self): return 2 * self.ROWS * self.COLS * 4
    def units(self): return self.ROWS * self.COLS
    def step(self, i): self.sets[i % len(self.sets)][0].run()


class C3SoftmaxWithArgmax(C3Softmax):
    """Softmax and row argmax of the same tensor as ONE equation: the arg reduction joins the first round of the row
    program, so x is read once for both results (reported beside the two separate operations)."""
    name = "c3_softmax_and_argmax_one_pass_fp32"
    description = "softmax rows + row argmax of fp32 [65536,4096] per GPU in one row program"

    def build(self, ex):
        x = ex.input("x")
        e = (x - x.reduce_max([1])).exp()
        return {"y": e / e.reduce_sum([1]), "idx": x.argmax([1], squeeze_axes=[1])}

    def algorithmic_bytes(self): return 2 * self.ROWS * self.COLS * 4 + self.ROWS * 4


class _ReferenceReduction:
    """One stamped launch of the REFERENCE's own reduction device code (oracle/_ref, baseline arms only): its CUB call or
    tiled kernel over a dense [outer, reduction, inner] input, workspace sized by its own query."""

    def __init__(self, op, x, out, outer, reduction, inner):
        import torch

        import oracle

        dt = {torch.float32: oracle.FP32, torch.float16: oracle.FP16, torch.bfloat16: oracle.BF16}
        self.args = (op, x, dt[x.dtype], out, dt[out.dtype], outer, reduction, inner)
        self.path, self.ws_bytes = oracle.reference_cub_reduce_workspace(op, dt[x.dtype], dt[out.dtype], outer, reduction, inner)
        self.ws = torch.empty(max(1, self.ws_bytes), dtype=torch.uint8, device="cuda")

    def run(self):
        import torch

        import oracle

        op, x, xd, out, od, outer, reduction, inner = self.args
        oracle.reference_cub_reduce(op, self.path, x.data_ptr(), xd, out.data_ptr(), od, outer, reduction, inner, self.ws.data_ptr(), self.ws_bytes,
                                    torch.cuda.current_stream().cuda_stream)


def _row_reduction_for_baseline(op, x, out, rows, cols):
    """(launcher, label): the reference's own reduction when oracle/_ref holds it, else ours standing in."""
    import oracle

    if oracle.reference_cub_reduce_lib() is not None:
        return _ReferenceReduction(op, x, out, rows, cols, 1), "reference CUB segmented reduce"
    from thor_b200.reductions import CubReduction, CubReductionOp

    ours = {"max": CubReductionOp.Max, "sum": CubReductionOp.Sum, "mean": CubReductionOp.Mean}[op]
    return CubReduction(ours, [1]).stamp(x, output=out), "rows reduction (ours)"


class C3ReferenceStagePipeline(C3Softmax):
    """Baseline, not product: the reference's stage list for the composed softmax -- Reduction(max), Fused(exp(x - m)),
    Reduction(sum), Fused(e / s) -- with the two fused stages being the kernels the reference's own emitter generates
    (oracle/_ref) and the two reductions its own CUB calls (cub::DeviceSegmentedReduce with its operators and iterators,
    compiled from its header into oracle/_ref; our row-reduction kernels stand in only where that library is not built).
    What the reference's pipeline costs on this GPU: four kernels, two materialised [rows, cols] fp32 intermediates."""
    is_baseline = True
    name = "c3_softmax_rows_fp32_reference_stage_list"
    description = "reference stage list for softmax: its emitted fused kernels + its CUB reductions (baseline beside c3)"

    def setup(self):
        import torch

        import oracle
        from oracle.refkernel import ReferenceBroadcastKernel
        from thor_b200.reductions import CubReduction, CubReductionOp

        if oracle.reference_emitter_lib() is None:
            raise RuntimeError("oracle/_ref/libthor_ref_emit.so is not built")
        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(77 + self.dist.rank)
        f32 = oracle.FP32
        self.k_exp = ReferenceBroadcastKernel("in:x in:m sub exp", {"x": f32, "m": f32}, {"x": (R, C), "m": (R, 1)})
        self.k_div = ReferenceBroadcastKernel("in:e in:s div", {"e": f32, "s": f32}, {"e": (R, C), "s": (R, 1)})
        self.x = torch.randn(R, C, device="cuda", generator=gen) * 3.0
        self.e = torch.empty(R, C, device="cuda")
        self.y = torch.empty(R, C, device="cuda")
        self.m = torch.empty(R, 1, device="cuda")
        self.s = torch.empty(R, 1, device="cuda")
        self.r_max, label = _row_reduction_for_baseline("max", self.x, self.m, R, C)
        self.r_sum, _ = _row_reduction_for_baseline("sum", self.e, self.s, R, C)
        self.sets = [None]  # one buffer set: 1 GiB per tensor, far beyond L2
        self.launches_per_step = 4
        self.kernel_kind = [label, "reference fused exp(x - m)", label, "reference fused e / s"]

    def step(self, i):
        self.r_max.run()
        self.k_exp.launch({"x": self.x, "m": self.m}, self.e)
        self.r_sum.run()
        self.k_div.launch({"e": self.e, "s": self.s}, self.y)


class C3Argmax(C3Softmax):
    name = "c3_row_argmax_fp32"
    description = "row argmax of fp32 [65536,4096] per GPU -> uint32 [65536]"

    def build(self, ex):
        return {"idx": ex.input("x").argmax([1], [1])}

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(78 + self.dist.rank)
        eq = ex.compile(self.build(ex))
        self.sets = []
        for _ in range(2):
            x = torch.randn(R, C, device="cuda", generator=gen) * 3.0
            self.sets.append((eq.stamp({"x": x}), x))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()

    def algorithmic_bytes(self): return self.ROWS * self.COLS * 4 + self.ROWS * 4


class C4FullReduce(Workload):
    name = "c4_full_reductions_bf16"
    description = "sum, sum of squares ((x*x).reduce_sum()) and max over bf16 n=2^31 per GPU, fp32 accumulation"
    dtype = "bf16->f32"
    N = 1 << 31

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        gen = torch.Generator(device="cuda").manual_seed(99 + self.dist.rank)
        self.x = torch.empty(self.N, device="cuda", dtype=torch.bfloat16)
        chunk = min(self.N, 1 << 28)
        for s in range(0, self.N, chunk):
            n = min(chunk, self.N - s)
            self.x[s:s + n] = (torch.randn(n, device="cuda", generator=gen) + 0.01).bfloat16()
        x = ex.input("x")
        eq = ex.compile({"sum": x.reduce_sum(), "sumsq": (x * x).reduce_sum(), "max": x.reduce_max()})
        self.plan = eq.stamp({"x": self.x})
        self.launches_per_step = self.plan.kernel_launches_per_run()
        self.kernel_kind = self.plan.physical_stage_names()
        self.outs = [self.plan.output(n) for n in ("sum", "sumsq", "max")]

    def algorithmic_bytes(self): return self.N * 2
    def units(self): return self.N
    def step(self, i):
        self.plan.run()
        if self.dist.enabled:
            # per-GPU fp32 partials -> one allreduce each (sum for the additive statistics, max for the maximum), on a side
            # stream: the collective of step i overlaps the kernel of step i + 1
            if not hasattr(self, "side"):
                self.side = _SideCollective()
            self.side.submit(sums=torch_cat(self.outs[:2]), maxima=self.outs[2].clone())

    def drain(self):
        if hasattr(self, "side"):
            self.side.drain()


class C3ArgmaxReferenceGpu(C3Argmax):
    """Baseline, not product: the reference's own row argmax -- cub::DeviceSegmentedReduce over its counting + transform
    iterator of {u64 index, float} candidates with its NaN-wins / lowest-index operator (oracle/_ref)."""
    is_baseline = True
    name = "c3_row_argmax_fp32_reference_gpu"
    description = "reference CUB arg reduction for the row argmax of fp32 [65536,4096] (baseline beside c3_argmax)"

    def setup(self):
        import torch

        import oracle

        lib_ = oracle.reference_cub_reduce_lib()
        if lib_ is None or not hasattr(lib_, "thor_ref_cub_argreduce"):
            raise RuntimeError("oracle/_ref holds no build of the reference's arg reductions")
        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(78 + self.dist.rank)
        self.path, self.ws_bytes = oracle.reference_cub_argreduce_workspace(True, oracle.FP32, R, C, 1, oracle.UINT32)
        self.ws = torch.empty(max(1, self.ws_bytes), dtype=torch.uint8, device="cuda")
        self.sets = []
        for _ in range(2):
            self.sets.append((torch.randn(R, C, device="cuda", generator=gen) * 3.0, torch.empty(R, dtype=torch.int32, device="cuda")))
        self.launches_per_step = 1
        self.kernel_kind = ["reference CUB segmented arg reduce"]

    def step(self, i):
        import torch

        import oracle

        x, idx = self.sets[i % len(self.sets)]
        oracle.reference_cub_argreduce(True, self.path, x.data_ptr(), oracle.FP32, 0, oracle.FP32, idx.data_ptr(), oracle.UINT32, self.ROWS, self.COLS, 1, self.ws.data_ptr(),
                                       self.ws_bytes, torch.cuda.current_stream().cuda_stream)


class C4ReferenceStagePipeline(C4FullReduce):
    """Baseline, not product: what the reference runs for the three statistics -- its full reduction (cub::DeviceReduce::
    TransformReduce with its fp32 operators) for the sum, its emitted flat kernel materialising x * x as bf16 followed by
    the same reduction for the sum of squares, and its NaN-propagating maximum: four kernels, three reads of x."""
    is_baseline = True
    name = "c4_full_reductions_bf16_reference_stage_list"
    description = "reference stage list for sum / sum of squares / max: its CUB full reductions + its emitted x*x kernel (baseline beside c4)"

    def setup(self):
        import torch

        import oracle
        from oracle.refkernel import ReferenceFlatKernel

        if oracle.reference_emitter_lib() is None or oracle.reference_cub_reduce_lib() is None:
            raise RuntimeError("oracle/_ref holds no build of the reference's emitter / reductions")
        gen = torch.Generator(device="cuda").manual_seed(99 + self.dist.rank)
        pad = 64
        self.x = torch.zeros(self.N + pad, device="cuda", dtype=torch.bfloat16)
        chunk = min(self.N, 1 << 28)
        for s in range(0, self.N, chunk):
            n = min(chunk, self.N - s)
            self.x[s:s + n] = (torch.randn(n, device="cuda", generator=gen) + 0.01).bfloat16()
        self.sq = torch.zeros(self.N + pad, device="cuda", dtype=torch.bfloat16)
        self.k_sq = ReferenceFlatKernel("in:x in:x mul", {"x": oracle.BF16}, self.N)
        self.outs = [torch.empty(1, device="cuda") for _ in range(3)]
        self.r_sum = _ReferenceReduction("sum", self.x, self.outs[0], 1, self.N, 1)
        self.r_sumsq = _ReferenceReduction("sum", self.sq, self.outs[1], 1, self.N, 1)
        self.r_max = _ReferenceReduction("max", self.x, self.outs[2], 1, self.N, 1)
        self.sets = [None]
        self.launches_per_step = 4
        self.kernel_kind = ["reference CUB transform-reduce (sum)", "reference fused x * x", "reference CUB transform-reduce (sum)", "reference CUB transform-reduce (max)"]

    def step(self, i):
        self.r_sum.run()
        self.k_sq.launch({"x": self.x}, self.sq)
        self.r_sumsq.run()
        self.r_max.run()


class _SideCollective:
    """Allreduce of a step's packed partials on a side stream, so that it overlaps the next step's kernel (the partials
    are packed on the main stream first, which also frees the step's output buffers for the next launch)."""

    def __init__(self):
        import torch

        self.stream = torch.cuda.Stream()

    def submit(self, **partials):
        import torch

        from thor_b200.sharding import combine_partials

        ready = torch.cuda.Event()
        ready.record()
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            combine_partials(**partials)
        for t in partials.values():
            t.record_stream(self.stream)

    def drain(self):
        import torch

        torch.cuda.current_stream().wait_stream(self.stream)


def torch_cat(ts):
    import torch

    return torch.cat([t.reshape(-1) for t in ts])


def _layernorm_expr(ex, eps=1e-5):
    from thor_b200 import DataType

    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    mean = x.reduce_mean([1])
    xc = x - mean
    var = (xc * xc).reduce_mean([1])
    rstd = 1.0 / (var + eps).sqrt()
    return (xc * rstd * gamma + beta).cast(DataType.bf16)


class C5LayerNormFwd(Workload):
    name = "c5_layernorm_forward_bf16"
    description = "Expression-authored LayerNorm forward over bf16 [32768,8192] per GPU (mean/var row reductions fused with the elementwise terms)"
    dtype = "bf16"
    ROWS, COLS = 32768, 8192

    def _inputs(self, gen):
        import torch

        R, C = self.ROWS, self.COLS
        x = torch.randn(R, C, device="cuda", generator=gen).bfloat16()
        gamma = (torch.rand(C, device="cuda", generator=gen) * 0.2 + 0.9).bfloat16()
        beta = (torch.randn(C, device="cuda", generator=gen) * 0.02).bfloat16()
        return x, gamma, beta

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        gen = torch.Generator(device="cuda").manual_seed(55 + self.dist.rank)
        eq = ex.compile({"y": _layernorm_expr(ex)}, row_program=ROW_PROGRAM)
        self.sets = []
        for _ in range(2):
            x, gamma, beta = self._inputs(gen)
            y = torch.empty_like(x)
            self.sets.append((eq.stamp({"x": x, "gamma": gamma, "beta": beta}, outputs={"y": y}), x, y))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()

    def algorithmic_bytes(self): return 2 * self.ROWS * self.COLS * 2 + 2 * self.COLS * 2
    def units(self): return self.ROWS * self.COLS
    def step(self, i): self.sets[i % len(self.sets)][0].run()


class C5FwdReferenceStagePipeline(C5LayerNormFwd):
    """Baseline, not product: the reference's stage list for the LayerNorm forward DAG -- Reduction(mean), Fused((x - mean)^2)
    into an fp32 [rows, cols] temporary, Reduction(mean), Fused(normalise, scale, shift, cast) -- with the reference's own
    emitted fused kernels and its own CUB reductions (ours stand in only where oracle/_ref holds no build of them)."""
    is_baseline = True
    name = "c5_layernorm_forward_bf16_reference_stage_list"
    description = "reference stage list for LayerNorm forward: its emitted fused kernels + its CUB reductions (baseline beside c5 forward)"

    def setup(self):
        import torch

        import oracle
        from oracle.refkernel import ReferenceBroadcastKernel
        from thor_b200 import DataType
        from thor_b200.reductions import CubReduction, CubReductionOp

        if oracle.reference_emitter_lib() is None:
            raise RuntimeError("oracle/_ref/libthor_ref_emit.so is not built")
        R, C = self.ROWS, self.COLS
        gen = torch.Generator(device="cuda").manual_seed(55 + self.dist.rank)
        self.x, self.gamma, self.beta = self._inputs(gen)
        f32, b16 = oracle.FP32, oracle.BF16
        self.k_sq = ReferenceBroadcastKernel("in:x in:mean sub in:x in:mean sub mul", {"x": b16, "mean": f32}, {"x": (R, C), "mean": (R, 1)})
        self.k_out = ReferenceBroadcastKernel("in:x in:mean sub lit:1 in:var lit:1e-05 add sqrt div mul in:gamma mul in:beta add cast:24",
                                              {"x": b16, "mean": f32, "var": f32, "gamma": b16, "beta": b16},
                                              {"x": (R, C), "mean": (R, 1), "var": (R, 1), "gamma": (C,), "beta": (C,)})
        self.sq = torch.empty(R, C, device="cuda", dtype=torch.float32)
        self.y = torch.empty(R, C, device="cuda", dtype=torch.bfloat16)
        self.mean = torch.empty(R, 1, device="cuda")
        self.var = torch.empty(R, 1, device="cuda")
        if oracle.reference_cub_reduce_lib() is not None:
            self.r_mean, label = _row_reduction_for_baseline("mean", self.x, self.mean, R, C)
        else:
            self.r_mean, label = CubReduction(CubReductionOp.Mean, [1], output_dtype=DataType.fp32).stamp(self.x, output=self.mean), "rows reduction (ours)"
        self.r_var, _ = _row_reduction_for_baseline("mean", self.sq, self.var, R, C)
        self.sets = [None]
        self.launches_per_step = 4
        self.kernel_kind = [label, "reference fused (x - mean)^2", label, "reference fused normalise"]

    def step(self, i):
        self.r_mean.run()
        self.k_sq.launch({"x": self.x, "mean": self.mean}, self.sq)
        self.r_var.run()
        self.k_out.launch({"x": self.x, "mean": self.mean, "var": self.var, "gamma": self.gamma, "beta": self.beta}, self.y)


class C5LayerNormBwd(C5LayerNormFwd):
    name = "c5_layernorm_backward_bf16"
    description = "autodiff-generated LayerNorm backward (dx, dgamma, dbeta) over bf16 [32768,8192] per GPU; dgamma/dbeta allreduced when N > 1"

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        gen = torch.Generator(device="cuda").manual_seed(56 + self.dist.rank)
        bwd = ex.compile({"y": _layernorm_expr(ex)}, row_program=ROW_PROGRAM).compile_backward(["x", "gamma", "beta"])
        self.sets = []
        for _ in range(2):
            x, gamma, beta = self._inputs(gen)
            dy = (torch.randn(self.ROWS, self.COLS, device="cuda", generator=gen) * 1e-2).bfloat16()
            plan = bwd.stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
            self.sets.append((plan, x, dy, torch_cat([plan.output("gamma_grad"), plan.output("beta_grad")])))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()

    def algorithmic_bytes(self): return 3 * self.ROWS * self.COLS * 2 + 3 * self.COLS * 2
    def step(self, i):
        plan = self.sets[i % len(self.sets)][0]
        plan.run()
        if self.dist.enabled:
            # the packed fp32 [dgamma, dbeta] partials are allreduced on a side stream, overlapping the next step's kernel
            if not hasattr(self, "side"):
                self.side = _SideCollective()
            self.side.submit(sums=torch_cat([plan.output("gamma_grad").float(), plan.output("beta_grad").float()]))

    def drain(self):
        if hasattr(self, "side"):
            self.side.drain()


WORKLOADS = {"c1": C1Cast, "c2": C2FusedExpr, "c3": C3Softmax, "c3_argmax": C3Argmax, "c3_both": C3SoftmaxWithArgmax, "c4": C4FullReduce, "c5_fwd": C5LayerNormFwd,
             "c5_bwd": C5LayerNormBwd, "c1_ref_gpu": C1CastReferenceGpu, "c2_ref_gpu": C2ReferenceGpu, "c3_ref_stages": C3ReferenceStagePipeline, "c3_argmax_ref_gpu": C3ArgmaxReferenceGpu, "c4_ref_stages": C4ReferenceStagePipeline,
             "c5_fwd_ref_stages": C5FwdReferenceStagePipeline}


# ---------------------------------------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------------------------------------
def reference_arm(args):
    """The reference's own CPU implementation of the path, on the host cores of this machine.

    The reference has a CPU path only for casts (TypeConverter::cpuConvertTypeImpl); its expressions and
    reductions exist on the GPU only, so for the headline workload (configuration 2) this arm times the
    CPU restatement of the reference's per-node arithmetic (oracle port), each step a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import oracle

    threads = oracle.host_threads()
    rows, cols = 512, 8192
    rng = np.random.default_rng(0)
    x = rng.standard_normal((rows, cols)).astype(np.float16)
    z = rng.standard_normal((rows, cols)).astype(np.float16)
    a = rng.uniform(0.5, 1.5, cols).astype(np.float16)
    bytes_per_step = 3 * rows * cols * 2 + cols * 2
    for _ in range(max(1, args.warmup)):
        oracle.c2_fused(a, x, 0.1, z, True, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.c2_fused(a, x, 0.1, z, True, threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = bytes_per_step / dt / 1e9
    sample = f"{rows} of 8192 rows x {cols} cols per step (oracle C port, OpenMP)"
    print(json.dumps({
        "impl": "reference", "metric": "fused_expr_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": {"workload": C2FusedExpr.name, "description": C2FusedExpr.description, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
    }))


def run_workload(dist: Dist, cls, steps: int, warmup: int, sample_clocks: bool, scale: float = 1.0):
    import thor_b200

    wl = cls(dist, scale)
    wl.setup()
    before = thor_b200.launch_count()
    sampler = ClockSampler(dist.local_rank if dist.enabled else 0) if (sample_clocks and dist.rank == 0) else None
    ms, wall, clocks = time_steps(dist, wl.step, steps, warmup, sampler, sample_clocks, getattr(wl, "drain", None))
    del before
    launches = wl.launches_per_step * steps  # kernels of this library inside the timed region
    return wl, ms, wall, clocks, launches


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations, the end-to-end leg and the CPU baseline")
    ap.add_argument("--scale", type=float, default=1.0, help="fraction of the workload's leading dimension (smaller cases for profiler captures only)")
    ap.add_argument("--row-program", default="", help="row-program layout fields, e.g. rows_per_iteration=1,ring_buffers=4 (comparison runs)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.row_program:
        global ROW_PROGRAM
        ROW_PROGRAM = {k: int(v) for k, v in (kv.split("=") for kv in args.row_program.split(","))}
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch

    import thor_b200

    dist = Dist(args.gpus)
    peak, peak_kind = measured_peak()
    wl, ms, wall, clocks, launches = run_workload(dist, WORKLOADS[args.workload], args.steps, args.warmup, True, args.scale)
    world = dist.world
    total_bytes = wl.algorithmic_bytes() * world
    value = total_bytes / (ms * 1e-3) / 1e9
    per_gpu_gbs = wl.algorithmic_bytes() / (ms * 1e-3) / 1e9
    line = {
        "metric": "fused_expr_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "description": wl.description, "sharding": f"rows x{world}, no collective" if world > 1 else "single GPU",
                   "cache": f"{len(wl.sets) or 1} rotating buffer sets, {wl.algorithmic_bytes() * max(1, len(wl.sets)) >> 20} MiB per GPU > 4 x L2",
                   "kernel": getattr(wl, "kernel_kind", None), "scale": args.scale},
        "elements_per_s": wl.units() * world / (ms * 1e-3),
        "wall_ms_per_step": wall,
        "clocks": clocks,
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": TRAFFIC_BYTES.get(wl.name), "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_launch": wl.algorithmic_bytes(),
                     "launch_us": ms * 1e3 / max(1, wl.launches_per_step)},
    }

    if not args.no_extras:
        # end to end: pinned host buffers -> H2D -> kernel -> D2H inside the timed region
        if hasattr(wl, "e2e_step") and not getattr(wl, "is_baseline", False):
            k = max(3, min(10, args.steps))
            e_ms, _, _ = time_steps(dist, wl.e2e_step, k, 3)
            h2d, d2h = wl.e2e_bytes()
            line["e2e"] = {"value": total_bytes / (e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": e_ms}
        # CPU baseline on rank 0 at N = 1: bounded sample of the same workload
        if world == 1 and hasattr(wl, "cpu_sample") and not getattr(wl, "is_baseline", False):
            import oracle

            threads = oracle.host_threads()
            wl.cpu_sample(64, threads)  # warm
            v, sample = wl.cpu_sample(1024, threads)
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample}
        del wl
        torch.cuda.empty_cache()
        extras = {}
        for key, cls in WORKLOADS.items():
            if key == args.workload:
                continue
            try:
                w2, ms2, _, _, l2 = run_workload(dist, cls, max(20, args.steps), 5, False)
                g = w2.algorithmic_bytes() / (ms2 * 1e-3) / 1e9
                extras[w2.name] = {"ms_per_step": ms2, "gbps_per_gpu": g, "gbps_total": g * world, "frac_of_peak": g / peak, "launches_per_step": w2.launches_per_step,
                                   "kernels": getattr(w2, "kernel_kind", None), "algorithmic_bytes": w2.algorithmic_bytes(),
                                   "elements_per_s": w2.units() * world / (ms2 * 1e-3)}
                del w2
                torch.cuda.empty_cache()
            except Exception as exc:  # a configuration that cannot run must not hide the headline number
                extras[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        line["all_configs"] = extras
    if dist.rank == 0:
        print(json.dumps(line))
    dist.close()


# DRAM bytes of the dominant kernel per launch, measured with ncu on a reduced case of the same kernel (one
# captured launch, summaries under profiles/) and scaled to the full launch by the elements processed: traffic
# grows in proportion (every input byte is read once).  Written bytes undercount outputs that are still dirty
# in the 126 MB L2 when a small case ends, so values below the algorithmic bytes mean "no re-reads", not less work.
TRAFFIC_BYTES = {
    "c1_cast_fp32_fp16": 71_600_000,                 # full size captured; most of the 33.5 MB output is still in L2 at kernel end
    "c2_fused_relu_axb_sigmoid": 2 * 161_700_000,    # 4096 of 8192 rows captured
    "c3_softmax_rows_fp32": 8 * 215_500_000,
    "c3_softmax_and_argmax_one_pass_fp32": 8 * 217_300_000,         # 8192 of 65536 rows captured
    "c3_row_argmax_fp32": 8 * 138_300_000,
    "c4_full_reductions_bf16": 16 * 272_400_000,     # 2^27 of 2^31 elements captured
    "c5_layernorm_forward_bf16": 8 * 78_900_000,     # 4096 of 32768 rows captured
    "c5_layernorm_backward_bf16": 8 * 170_100_000,
    "c2_fused_relu_axb_sigmoid_reference_gpu_kernel": 2 * 173_900_000,
}

if __name__ == "__main__":
    main()
