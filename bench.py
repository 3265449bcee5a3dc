#!/usr/bin/env python
"""Benchmark of the hot path: fused expression / reduction / cast kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2] [--no-extras]

A step is one pass of the hot path over one batch of synthetic input resident in HBM.  The headline workload is
configuration 2 (y = relu(a*x + b) * sigmoid(z), fp16 [8192, 8192], a per column, b an fp32 runtime scalar).  With N > 1
the FIXED global problem of every configuration is sharded along its leading dimension (rows / flat index) over the N
ranks -- strong scaling: `value` is the global problem's algorithmic bytes over the slowest rank's time.  Elementwise,
cast and row-wise configurations need no communication; the full reductions (configuration 4) and the LayerNorm
dgamma / dbeta column sums (configuration 5 backward) combine per-GPU fp32 partials with one NCCL allreduce per step
through the library's own communicator, inside the timed region, and the combined results are checked against the CPU
oracle of the global problem after the timed region ("multi_gpu_check").  Every configuration is reported under
roofline.per_config (time per step, fraction of the HBM roofline per GPU, at N > 1 the allreduce timed alone and the
1-GPU time of the same global problem measured on rank 0 in the same run); "all_configs" carries the detail.

Timing: W >= 3 warm-up steps, then exactly K steps between a barrier + synchronize on both sides, bracketed by CUDA events
on the launching stream; the max over ranks is reported.  Buffers rotate over several disjoint sets whose total size is
several times the 126 MB L2, so no step finds its inputs in cache.  After the timed region the same load keeps running in
11 timed groups (at least 400 ms in all) while nvidia-smi samples SM clocks and throttle reasons: roofline.sustained holds
the median / p10 / p90 per-step time of those groups and roofline.frac_sustained the fraction at the clocks that were
sampled.

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

    def communicator(self):
        """The library's own NCCL communicator (thor_b200_comm_*) over the ranks of this job; the id travels through the
        process group that torchrun set up.  Data-path collectives of the benchmark go through it."""
        if not self.enabled:
            return None
        if getattr(self, "_comm", None) is None:
            import torch

            from thor_b200.sharding import Communicator

            uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if self.rank == 0:
                uid.copy_(torch.frombuffer(bytearray(Communicator.unique_id()), dtype=torch.uint8))
            self.dist.broadcast(uid, src=0)
            self._comm = Communicator(self.world, self.rank, bytes(uid.cpu().numpy().tobytes()))
        return self._comm

    def sum_f64(self, values):
        """Sum / of float64 host values over the ranks (oracle partials of the result check)."""
        import torch

        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        if self.enabled:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t.cpu().numpy()

    def max_f64(self, values):
        import torch

        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        if self.enabled:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.cpu().numpy()

    def close(self):
        if getattr(self, "_comm", None) is not None:
            self._comm.close()
        if self.enabled:
            self.dist.destroy_process_group()


class SingleRank:
    """Stands in for Dist when rank 0 times the WHOLE global problem alone (the 1-GPU time of the strong-scaling ratio)."""
    enabled, world, rank = False, 1, 0

    def __init__(self, local_rank):
        self.local_rank = local_rank

    def barrier(self):
        import torch

        torch.cuda.synchronize()

    def max(self, v): return v
    def communicator(self): return None


def time_steps(dist, step, steps: int, warmup: int, drain=None):
    """W untimed + K timed calls of step(i).  Returns {"ms": device ms per step (max over ranks), "wall_ms": host ms per step,
    "launches": kernels this library launched inside the timed region (read from its own counter)}.  `drain` makes the timing
    stream wait for work the steps put on side streams, so that it ends inside the timed region."""
    import torch

    import thor_b200

    for i in range(warmup):
        step(i)
    if drain is not None:
        drain()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = thor_b200.launch_count()
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        step(warmup + i)
    if drain is not None:
        drain()
    e1.record()
    issued = (time.perf_counter() - t0) * 1e3 / steps
    launches = thor_b200.launch_count() - before
    dist.barrier()
    return {"ms": dist.max(e0.elapsed_time(e1) / steps), "host_issue_ms": dist.max(issued), "launches": int(launches)}


def time_sustained(dist, step, steps: int, first: int, ms_hint: float, sampler: ClockSampler | None, drain=None, groups: int = 11, min_total_ms: float = 1500.0):
    """The same load kept running after the timed region: `groups` groups of equal length, each bracketed by its own event
    pair, at least min_total_ms in all (nvidia-smi cannot sample faster than every ~20 ms).  Every rank derives the group
    length from the rank-maximum time of the timed region, so collectives stay matched.  Returns per-step statistics over
    the groups (rank maximum per group) and the clocks sampled while they ran."""
    import torch

    per_group = max(steps, int(min_total_ms / groups / max(ms_hint, 1e-4)) + 1)
    if sampler:
        sampler.start()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(groups + 1)]
    i = first
    events[0].record()
    for g in range(groups):
        for _ in range(per_group):
            step(i)
            i += 1
        if drain is not None:
            drain()
        events[g + 1].record()
    dist.barrier()
    times = sorted(dist.max(events[g].elapsed_time(events[g + 1]) / per_group) for g in range(groups))
    clocks = sampler.stop() if sampler else None
    pick = lambda q: times[min(groups - 1, max(0, int(round(q * (groups - 1)))))]
    return {"groups": groups, "steps_per_group": per_group, "ms_median": pick(0.5), "ms_p10": pick(0.1), "ms_p90": pick(0.9)}, clocks


# ---------------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    description = ""
    dtype = ""
    unit_name = "elements"

    def __init__(self, dist, scale: float = 1.0):
        from thor_b200.sharding import shard_range

        self.dist = dist
        self.scale = scale  # fraction of the leading dimension (profiling captures use a smaller case)
        self.sets = []
        self.launches_per_step = 0
        # ROWS / N of the class is the GLOBAL problem; the instance works on this rank's contiguous shard of it
        self.lead = "ROWS" if hasattr(self, "ROWS") else "N"
        total = getattr(type(self), self.lead)
        if scale != 1.0:
            total = max(8, int(total * scale) // 8 * 8)
        self.global_lead = total
        self.shard = shard_range(total, dist.rank, dist.world, 8 if self.lead == "N" else 1)
        setattr(self, self.lead, self.shard[1] - self.shard[0])

    def algorithmic_bytes(self) -> int: raise NotImplementedError
    def units(self) -> int: raise NotImplementedError
    def setup(self): raise NotImplementedError
    def step(self, i: int): raise NotImplementedError

    def _of_global(self, fn):
        local = getattr(self, self.lead)
        setattr(self, self.lead, self.global_lead)
        try:
            return fn()
        finally:
            setattr(self, self.lead, local)

    def global_algorithmic_bytes(self) -> int: return self._of_global(self.algorithmic_bytes)
    def global_units(self) -> int: return self._of_global(self.units)

    def n_sets(self, bytes_per_set: int) -> int:
        return max(2, min(16, -(-4 * L2_BYTES // max(1, bytes_per_set))))

    def sharding(self) -> str:
        if self.dist.world == 1:
            return "single GPU"
        return f"{self.lead.lower()} {self.global_lead} split over {self.dist.world} ranks ({getattr(self, self.lead)} on this rank), {self.collective}"

    collective = "no collective"


class C1Cast(Workload):
    name = "c1_cast_fp32_fp16"
    description = "TypeConverter fp32->fp16, 1-D, n=2^24, U(-4,4) with edge values at 0.1%"
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
        # the cast of a shard takes a few microseconds: the timed loop runs stamped conversions (one C call each)
        self.stamped = [TypeConverter.stamp(src, dst) for src, dst in self.sets]
        self.launches_per_step = 1
        self.host_in = host.pin_memory()
        self.host_out = torch.empty(self.n, dtype=torch.float16).pin_memory()

    def algorithmic_bytes(self): return self.N * 6
    def units(self): return self.N
    def step(self, i): self.stamped[i % len(self.stamped)].run()

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

    def step(self, i):
        src, dst = self.sets[i % len(self.sets)]
        self.convert(src, dst)


class C2FusedExpr(Workload):
    name = "c2_fused_relu_axb_sigmoid"
    description = "y = relu(a*x + b) * sigmoid(z): x,z,y fp16 [8192,8192], a fp16 [8192] per column, b fp32 runtime scalar 0.1"
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
    description = "exp(x - max_row) / sum_row(exp(x - max_row)) on fp32 [65536,4096] (composed expression)"
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
    description = "softmax rows + row argmax of fp32 [65536,4096] in one row program"

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
    description = "row argmax of fp32 [65536,4096] -> uint32 [65536]"

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


class _ShardCombiner:
    """Combines this rank's fp32 partials with the other ranks' through the library's overlapped combiner
    (thor_b200_combiner_*: one NCCL group per step on a high-priority stream of its own).  The partial buffers are
    double-buffered with the plans that write them, so the collective of step i overlaps the kernel of step i + 1; a
    buffer's next kernel waits for that buffer's last collective."""

    def __init__(self, comm, buffers: int):
        from thor_b200.sharding import Combiner

        self.comm = comm
        self.native = Combiner(comm, buffers)
        self.stream = self.native.stream

    # Three slots, not two: a persistent kernel fills every SM, so the collective of step i only gets to run when the kernel of
    # step i + 1 drains; with two slots the kernel of step i + 2 would wait for it at every boundary (measured at N = 2,
    # LayerNorm backward: 177 us per step against 156 us), with three it never does.
    SLOTS = 3

    def bind(self, b: int, sums=None, maxima=None, rounded=None):
        """Slot b with its buffers resolved once: .wait() before the step's kernels, .submit() after them (one C call each)."""
        return self.native.bind(b, sums=sums, maxima=maxima, rounded_sums=rounded)

    def drain(self): self.native.drain()

    def time_alone(self, dist, sums=None, maxima=None, iters: int = 50) -> float:
        """Microseconds of one collective with nothing else on the GPU (events around `iters` back-to-back calls on the
        combiner's stream, max over ranks): the NVLink time of the step."""
        import torch

        scratch_s = sums.clone() if sums is not None else None
        scratch_m = maxima.clone() if maxima is not None else None
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(5):
            self.comm.allreduce_stats(sums=scratch_s, maxima=scratch_m, stream=self.stream)
        e0.record(self.stream)
        for _ in range(iters):
            self.comm.allreduce_stats(sums=scratch_s, maxima=scratch_m, stream=self.stream)
        e1.record(self.stream)
        self.stream.synchronize()
        return dist.max(e0.elapsed_time(e1) / iters * 1e3)


class C4FullReduce(Workload):
    name = "c4_full_reductions_bf16"
    description = "sum, sum of squares ((x*x).reduce_sum()) and max over bf16 n=2^31, fp32 accumulation"
    dtype = "bf16->f32"
    N = 1 << 31
    collective = "per-GPU {sum, sum of squares} and {max} combined in one NCCL group per step"
    combiner = None

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
        # one stamped plan per combiner slot over the same input, each with its own [sum, sumsq, max] fp32 result buffer
        self.stats = [torch.zeros(3, device="cuda") for _ in range(_ShardCombiner.SLOTS)]
        self.plans = [eq.stamp({"x": self.x}, outputs={"sum": st[0:1], "sumsq": st[1:2], "max": st[2:3]}) for st in self.stats]
        self.sets = self.plans
        self.launches_per_step = self.plans[0].kernel_launches_per_run()
        self.kernel_kind = self.plans[0].physical_stage_names()
        comm = self.dist.communicator()
        self.combiner = _ShardCombiner(comm, _ShardCombiner.SLOTS) if comm is not None else None
        self.slots = [self.combiner.bind(b, sums=st[0:2], maxima=st[2:3]) for b, st in enumerate(self.stats)] if self.combiner else None

    def algorithmic_bytes(self): return self.N * 2
    def units(self): return self.N
    def step(self, i):
        b = i % _ShardCombiner.SLOTS
        if self.combiner is None:
            self.plans[b].run()
            return
        self.slots[b].wait()
        self.plans[b].run()
        self.slots[b].submit()

    def drain(self):
        if self.combiner is not None:
            self.combiner.drain()

    def collective_us(self):
        return self.combiner.time_alone(self.dist, sums=self.stats[0][0:2].clone(), maxima=self.stats[0][2:3].clone()) if self.combiner else None

    def check(self):
        """The combined statistics against the CPU oracle of the GLOBAL problem: every rank's host cores reduce its own shard
        in float64, the float64 partials are added / maximised across the ranks."""
        import torch

        import oracle

        self.step(0)
        self.drain()
        torch.cuda.synchronize()
        got = self.stats[0].cpu().numpy().astype("float64")
        s, q, m = oracle.c4_stats(self.x.view(torch.uint16).cpu().numpy())
        s, q = self.dist.sum_f64([s, q]) if self.dist.enabled else (s, q)
        m = float(self.dist.max_f64([m])[0]) if self.dist.enabled else m
        n = self.global_lead
        ok = abs(got[0] - s) <= 1e-5 * abs(s) + 2e-7 * n and abs(got[1] - q) <= 1e-5 * abs(q) and got[2] == m
        return bool(ok), f"sum {got[0]:.6g} vs {s:.6g}, sumsq {got[1]:.6g} vs {q:.6g}, max {got[2]:.6g} vs {m:.6g}"


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
    description = "Expression-authored LayerNorm forward over bf16 [32768,8192] (mean/var row reductions fused with the elementwise terms)"
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
    description = ("autodiff-generated LayerNorm backward (dx, dgamma, dbeta) over bf16 [32768,8192]; per-GPU fp32 dgamma/dbeta sums allreduced "
                   "and rounded once when N > 1")
    collective = "per-GPU fp32 [2, 8192] dgamma / dbeta sums combined by one allreduce per step, rounded to bf16 once after it"
    combiner = None

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        gen = torch.Generator(device="cuda").manual_seed(56 + self.dist.rank)
        sharded = self.dist.enabled
        tuning = dict(ROW_PROGRAM or {})
        if self.dist.world >= 8 and "reserve_sms" not in tuning:
            # Eight ranks: the shard's kernel takes about 40 us and the collective about 26 us; a persistent grid over every
            # SM leaves the collective's CTAs nowhere to run until it drains.  Measured per step at N = 8 with 0 / 4 / 8 / 16 /
            # 32 SMs left free: 61.8 / 54.2 / 57.8 / 56.9 / 61.7 us.  At N = 2 it made no difference, so it stays 0 there.
            tuning["reserve_sms"] = 4
        bwd = ex.compile({"y": _layernorm_expr(ex)}, row_program=tuning or None, unrounded_column_sums=sharded).compile_backward(["x", "gamma", "beta"])
        self.sets = []
        for _ in range(_ShardCombiner.SLOTS if sharded else 2):
            x, gamma, beta = self._inputs(gen)
            dy = (torch.randn(self.ROWS, self.COLS, device="cuda", generator=gen) * 1e-2).bfloat16()
            plan = bwd.stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
            grads = torch.empty(2, self.COLS, device="cuda", dtype=torch.bfloat16) if sharded else None  # the combined gradients
            self.sets.append((plan, x, dy, gamma, plan.output("__column_sums") if sharded else None, grads))
        self.launches_per_step = self.sets[0][0].kernel_launches_per_run()
        self.kernel_kind = self.sets[0][0].physical_stage_names()
        comm = self.dist.communicator()
        self.combiner = _ShardCombiner(comm, _ShardCombiner.SLOTS) if comm is not None else None
        # the unrounded fp32 sums of this rank's rows are added across the ranks, then rounded to the gradients' dtype once
        self.slots = [self.combiner.bind(b, sums=st[4], rounded=st[5]) for b, st in enumerate(self.sets)] if self.combiner else None

    def algorithmic_bytes(self): return 3 * self.ROWS * self.COLS * 2 + 3 * self.COLS * 2
    def step(self, i):
        b = i % len(self.sets)
        plan, _, _, _, sums, grads = self.sets[b]
        if self.combiner is None:
            plan.run()
            return
        self.slots[b].wait()
        plan.run()
        self.slots[b].submit()

    def drain(self):
        if self.combiner is not None:
            self.combiner.drain()

    def collective_us(self):
        return self.combiner.time_alone(self.dist, sums=self.sets[0][4].clone()) if self.combiner else None

    def check(self):
        """dgamma / dbeta of the GLOBAL problem: every rank's host cores compute the float64 column sums of its own rows
        (the oracle's LayerNorm backward), the float64 partials are added across the ranks and compared with the allreduced,
        once-rounded bf16 gradients; dx is compared on a sample of this rank's rows."""
        import numpy as np
        import torch

        import oracle
        from oracle import expr_oracle as eo

        self.step(0)
        self.drain()
        torch.cuda.synchronize()
        plan, x, dy, gamma, sums, grads = self.sets[0]
        u16 = lambda t: t.contiguous().view(torch.uint16).cpu().numpy()
        want_dx, dg, db = oracle.layernorm_bwd(u16(x), u16(gamma), u16(dy), 1e-5)
        want = np.concatenate([dg, db])
        if self.dist.enabled:
            want = self.dist.sum_f64(want.tolist())
            got = grads.float().cpu().numpy().astype(np.float64).reshape(-1)
        else:
            got = np.concatenate([plan.output("gamma_grad").float().cpu().numpy().reshape(-1), plan.output("beta_grad").float().cpu().numpy().reshape(-1)]).astype(np.float64)
        rows_global = self.global_lead
        d = eo.ulp_distance(got, eo.round_to(want, oracle.BF16), oracle.BF16)
        d = np.where(np.abs(got - want) <= 1e-5 * np.abs(want) + 2e-7 * rows_global * 1e-2 + 2.0 ** -9 * np.abs(want), 0.0, d)
        sample = slice(0, min(64, self.ROWS))
        got_dx = plan.output("x_grad")[sample].float().cpu().numpy().astype(np.float64).reshape(-1)
        w_dx = oracle.to_float64(want_dx[sample].reshape(-1), oracle.BF16)
        ddx = eo.ulp_distance(got_dx, w_dx, oracle.BF16)
        ddx = np.where(np.abs(got_dx - w_dx) <= 2e-8, 0.0, ddx)
        ok = float(d.max()) <= 1.0 and float(ddx.max()) <= 1.0
        return bool(ok), f"dgamma/dbeta max {float(d.max()):.2f} bf16 ulp beyond tolerance, dx max {float(ddx.max()):.2f} ulp"



class C5BwdStageList(C5LayerNormBwd):
    """Baseline, not product: the reference's stage cut of the autodiff LayerNorm backward -- every reduction a stage of its
    own, fused kernels between them, the fp32 [rows, cols] intermediates materialised in HBM (ten stages, twelve launches)
    -- run with THIS library's fused and reduction kernels, which are at least as fast as the reference's own (see the
    other reference baselines), so the ratio to the row program understates the reference's cost rather than inflating
    it.  The reference's own emitted kernels are not used here because its multi-output fused stages cannot be driven
    through the single-output launcher of the test infrastructure."""
    is_baseline = True
    name = "c5_layernorm_backward_bf16_reference_stage_cut_own_kernels"
    description = ("reference stage cut for the autodiff LayerNorm backward (Reduction / FusedKernel stages with materialised fp32 intermediates), "
                   "this library's kernels per stage (baseline beside c5 backward)")
    collective = None

    def setup(self):
        import torch

        from thor_b200.expression import Expression as ex

        gen = torch.Generator(device="cuda").manual_seed(56 + self.dist.rank)
        bwd = ex.compile({"y": _layernorm_expr(ex)}, fuse_row_reductions=False).compile_backward(["x", "gamma", "beta"])
        x, gamma, beta = self._inputs(gen)
        dy = (torch.randn(self.ROWS, self.COLS, device="cuda", generator=gen) * 1e-2).bfloat16()
        plan = bwd.stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
        self.sets = [(plan, x, dy, gamma, None, None)]
        self.launches_per_step = plan.kernel_launches_per_run()
        self.kernel_kind = plan.physical_stage_names()
        self.combiner = None

    def step(self, i): self.sets[0][0].run()
    def collective_us(self): return None



class C5BwdReferenceKernels(C5LayerNormBwd):
    """Baseline, not product: the autodiff LayerNorm backward as the REFERENCE would run it.  The backward graph is the one
    the reference's own buildBackwardOutputs builds (tests/golden/autodiff_reference_graphs.json, dumped from its AutoDiff.cpp);
    oracle/stage_cut.py cuts it by the reference's planning rule (every reduction a stage over a tensor in memory, fused
    stages between them); every fused stage is the kernel the reference's own emitter generates for it and every reduction its
    own CUB call or tiled kernel (oracle/_ref).  One fused kernel per materialised tensor: where the reference would put two
    outputs into one kernel this re-reads their shared inputs, which matters little next to the two column sums
    ([1, 32768, 8192] over axis 0: its tiled kernel walks them on two CTAs)."""
    is_baseline = True
    name = "c5_layernorm_backward_bf16_reference_kernels"
    description = ("reference stage list for the autodiff LayerNorm backward: its own backward graph cut by its planning rule, its emitted fused kernels + "
                   "its CUB / tiled reductions (baseline beside c5 backward)")
    collective = None

    def setup(self):
        import torch

        import oracle
        from oracle import stage_cut
        from oracle.refkernel import ReferenceBroadcastKernel
        from thor_b200.dtypes import DataType, to_torch

        if oracle.reference_emitter_lib() is None or oracle.reference_cub_reduce_lib() is None:
            raise RuntimeError("oracle/_ref holds no build of the reference's emitter / reductions")
        R, C = self.ROWS, self.COLS
        golden = json.loads((ROOT / "tests" / "golden" / "autodiff_reference_graphs.json").read_text())["layernorm_bf16_32768x8192"]
        graph = stage_cut.merge_equal_nodes(golden["graph"])
        shapes = {"x": (R, C), "gamma": (C,), "beta": (C,), "__grad_output": (R, C)}
        gen = torch.Generator(device="cuda").manual_seed(56 + self.dist.rank)
        x, gamma, beta = self._inputs(gen)
        dy = (torch.randn(R, C, device="cuda", generator=gen) * 1e-2).bfloat16()
        self.tensors = {"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy}
        dtype_of = {"x": oracle.BF16, "gamma": oracle.BF16, "beta": oracle.BF16, "__grad_output": oracle.BF16}
        self.stages, self.kernel_kind = [], []
        for st in stage_cut.stage_list(graph, shapes):
            out = torch.empty(st["shape"], device="cuda", dtype=to_torch(DataType(st["dtype"])))
            self.tensors[st["name"]], dtype_of[st["name"]] = out, st["dtype"]
            if st["kind"] == "reduction":
                src = self.tensors[st["input"]]
                rows, cols = st["input_shape"]
                outer, n, inner = (rows, cols, 1) if st["axes"] == [1] else (1, rows, cols)
                red = _ReferenceReduction(st["op"], src, out, outer, n, inner)
                self.stages.append(red.run)
                self.kernel_kind.append(f"reference reduction {st['op']} over axis {st['axes'][0]} -> {st['name']}")
            else:
                dims = {name: tuple(self.tensors[name].shape) for name in st["inputs"]}
                dts = {name: dtype_of[name] for name in st["inputs"]}
                kernel = ReferenceBroadcastKernel(st["program"], dts, dims)
                if kernel.out_dtype != st["dtype"]:  # the graph stores this node in another dtype than the expression resolves to on its own
                    kernel = ReferenceBroadcastKernel(st["program"] + f" cast:{st['dtype']}", dts, dims)
                ins = {name: self.tensors[name] for name in st["inputs"]}
                self.stages.append(lambda k=kernel, i=ins, o=out: k.launch(i, o))
                self.kernel_kind.append(f"reference fused -> {st['name']}")
        self.sets = [None]
        self.launches_per_step = len(self.stages)
        self.combiner = None
        # sanity: the baseline computes the same gradients as the row program (same inputs), or it times nothing useful
        from thor_b200.expression import Expression as ex

        self.step(0)
        ours = ex.compile({"y": _layernorm_expr(ex)}).compile_backward(["x", "gamma", "beta"]).stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
        ours.run()
        torch.cuda.synchronize()
        for name in ("x_grad", "gamma_grad", "beta_grad"):
            a, b = self.tensors[name].float().reshape(-1), ours.output(name).float().reshape(-1)
            worst = float((a - b).abs().max() / (b.abs().max() + 1e-30))
            if not worst < 2e-2:
                raise RuntimeError(f"reference-kernel baseline disagrees with the row program on {name}: {worst:.3e} of the largest value")
        del ours

    def step(self, i):
        for run in self.stages:
            run()

    def collective_us(self): return None

class F3ScatterAdd(Workload):
    """Flat scatter-add without atomics (the step behind arg scans in scan min / max backward): 2^24 fp32 updates with
    uniformly random uint32 destinations into 2^20 outputs, duplicates added in update order.  Algorithmic bytes = one
    read of updates and destinations + one write of the output; the stable radix sort behind it moves 24 bytes per
    update and pass on top, which is what bounds it.  One GPU only (shards of the updates would need the outputs added)."""
    single_gpu_only = True
    name = "f3_flat_scatter_add_fp32"
    description = "flat scatter-add, 2^24 fp32 updates with random uint32 destinations into 2^20 outputs, no atomics, update order kept"
    dtype = "f32"
    N = 1 << 24
    OUT = 1 << 20

    def setup(self):
        import torch

        from thor_b200.reductions import FlatScatterAdd

        gen = torch.Generator(device="cuda").manual_seed(77)
        self.sets = []
        for _ in range(2):
            u = torch.randn(self.N, device="cuda", generator=gen)
            i = torch.randint(0, self.OUT, (self.N,), device="cuda", generator=gen).to(torch.uint32)
            self.sets.append((u, i, torch.empty(self.OUT, device="cuda")))
        self.plan = FlatScatterAdd(*self.sets[0])
        self.launches_per_step = self.plan.kernel_launches
        self.kernel_kind = ["digitHistogramKernel", "tableScanKernel", "digitScatterKernel", "applyRunsKernel"]

    def algorithmic_bytes(self): return self.N * 8 + self.OUT * 4
    def units(self): return self.N
    def step(self, i):
        u, idx, out = self.sets[i % len(self.sets)]
        self.plan.run(u, idx, out)

WORKLOADS = {"c1": C1Cast, "c2": C2FusedExpr, "c3": C3Softmax, "c3_argmax": C3Argmax, "c3_both": C3SoftmaxWithArgmax, "c4": C4FullReduce, "c5_fwd": C5LayerNormFwd,
             "c5_bwd": C5LayerNormBwd, "c1_ref_gpu": C1CastReferenceGpu, "c2_ref_gpu": C2ReferenceGpu, "c3_ref_stages": C3ReferenceStagePipeline, "c3_argmax_ref_gpu": C3ArgmaxReferenceGpu, "c4_ref_stages": C4ReferenceStagePipeline,
             "c5_fwd_ref_stages": C5FwdReferenceStagePipeline, "c5_bwd_ref_stages": C5BwdReferenceKernels, "c5_bwd_stage_cut": C5BwdStageList, "f3_scatter": F3ScatterAdd}


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
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": {"workload": C2FusedExpr.name, "description": C2FusedExpr.description, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
    }))


def load_traffic():
    """DRAM bytes per launch of each workload's dominant kernel, from the committed summary of the ncu captures
    (profiles/traffic.json: read and written bytes of ONE captured launch of a reduced case and the fraction of the full
    workload that case is; traffic grows in proportion because every input byte is read exactly once)."""
    try:
        return json.loads((ROOT / "profiles" / "traffic.json").read_text())
    except Exception:
        return {}


def traffic_of(table, wl):
    t = table.get(wl.name)
    if not t:
        return None, None
    k = 1.0 / float(t.get("fraction_of_workload", 1.0))
    total = (t["dram_read_bytes"] + t["dram_write_bytes"]) * k
    read_ratio = t["dram_read_bytes"] * k / max(1, t.get("algorithmic_read_bytes_full", 0)) if t.get("algorithmic_read_bytes_full") else None
    return total, read_ratio


def measure(dist, cls, steps: int, warmup: int, scale: float, sustained: bool, sampler=None):
    """Sets the workload up on this rank's shard and times it.  Returns (workload, result dict)."""
    wl = cls(dist, scale)
    wl.setup()
    drain = getattr(wl, "drain", None)
    r = time_steps(dist, wl.step, steps, warmup, drain)
    if sustained:
        stats, clocks = time_sustained(dist, wl.step, steps, warmup + steps, r["ms"], sampler, drain)
        r["sustained"], r["clocks"] = stats, clocks
    return wl, r


def config_entry(wl, r, peak, world):
    per_gpu = wl.algorithmic_bytes() / (r["ms"] * 1e-3) / 1e9  # this rank's shard over the slowest rank's time
    e = {"us": round(r["ms"] * 1e3, 3), "frac": round(per_gpu / peak, 4), "gbps_total": round(wl.global_algorithmic_bytes() / (r["ms"] * 1e-3) / 1e9, 1),
         "launches": round(r["launches"] / max(1, r["steps"]), 2)}
    if "sustained" in r:
        e["us_sustained_median"] = round(r["sustained"]["ms_median"] * 1e3, 3)
    return e


def one_gpu_time(dist, cls, steps: int, warmup: int, scale: float):
    """Microseconds per step of the WHOLE global problem on one GPU, measured by rank 0 alone while the other ranks wait:
    the T(1) of the strong-scaling ratio, from the same run and the same box."""
    import torch

    us = 0.0
    if dist.rank == 0:
        alone = SingleRank(dist.local_rank)
        w1 = cls(alone, scale)
        w1.setup()
        us = time_steps(alone, w1.step, steps, warmup, getattr(w1, "drain", None))["ms"] * 1e3
        del w1
        torch.cuda.empty_cache()
    dist.barrier()
    return dist.max(us)


def c1_cpu_reference(n: int):
    """The reference's own CPU converter (TypeConverter::cpuConvertTypeImpl compiled from its checkout into oracle/_ref) on
    the full 2^24-element input with its own thread rule, min(processors, n / 500000) (TypeConverter.cpp:919-925)."""
    import numpy as np

    import oracle
    from thor_b200.workloads import cast_input

    if oracle.reference_cast_lib() is None:
        return None
    x = cast_input(n, seed=0)
    oracle.reference_cast(x[: 1 << 20], oracle.FP32, oracle.FP16)
    best = None
    for _ in range(5):
        t0 = time.perf_counter()
        oracle.reference_cast(x, oracle.FP32, oracle.FP16)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": n * 6 / best / 1e9, "unit": "GB/s", "cores": int(oracle.reference_cast_lib().thor_ref_omp_threads_for(n)), "kind": "reference",
            "sample": f"all {n} elements, best of 5 passes of the reference's cpuConvertTypeImpl"}


def extras(args, dist, wl, line, per_config, peak, traffic):
    """Everything beside the headline's device-timed number: its end-to-end leg and CPU baseline, the strong-scaling 1-GPU
    time, every other configuration, the reference's GPU baselines (one GPU only) and the check of the combined results."""
    import torch

    world = dist.world
    steps = max(20, args.steps)
    checks = {}

    def finish(key, cls, w, entry):
        if world > 1:
            coll = w.collective_us() if hasattr(w, "collective_us") else None
            if coll is not None:
                entry["allreduce_us"] = round(coll, 2)
            if hasattr(w, "check"):
                ok, detail = w.check()
                ok = bool(dist.max(0.0 if ok else 1.0) == 0.0)
                checks[w.name] = "ok" if ok else "MISMATCH: " + detail
                entry["check"] = checks[w.name]
        return entry

    # end to end: pinned host buffers -> H2D -> kernel -> D2H inside the timed region, through the public API
    if hasattr(wl, "e2e_step") and not getattr(wl, "is_baseline", False):
        k = max(3, min(10, args.steps))
        e = time_steps(dist, wl.e2e_step, k, 3)
        h2d, d2h = wl.e2e_bytes()
        line["e2e"] = {"value": wl.global_algorithmic_bytes() / (e["ms"] * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "ms_per_step": e["ms"]}
    if world == 1 and hasattr(wl, "cpu_sample") and not getattr(wl, "is_baseline", False):
        import oracle

        threads = oracle.host_threads()
        wl.cpu_sample(64, threads)  # warm
        v, sample = wl.cpu_sample(1024, threads)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample}
    finish(args.workload, WORKLOADS[args.workload], wl, per_config[wl.name])
    del wl
    torch.cuda.empty_cache()
    if world > 1:
        t1 = one_gpu_time(dist, WORKLOADS[args.workload], steps, 5, args.scale)
        first = per_config[next(iter(per_config))]
        first["one_gpu_us"], first["speedup"] = round(t1, 3), round(t1 / first["us"], 3)

    detail = {}
    for key, cls in WORKLOADS.items():
        if key == args.workload or (world > 1 and (getattr(cls, "is_baseline", False) or getattr(cls, "single_gpu_only", False))):
            continue
        try:
            w2, r2 = measure(dist, cls, steps, 5, 1.0, False)
            r2["steps"] = steps
            entry = config_entry(w2, r2, peak, world)
            t_bytes, read_ratio = traffic_of(traffic, w2)
            detail[w2.name] = {"description": w2.description, "sharding": w2.sharding(), "kernels": getattr(w2, "kernel_kind", None),
                               "algorithmic_bytes_per_gpu": w2.algorithmic_bytes(), "elements_per_s": w2.global_units() / (r2["ms"] * 1e-3),
                               "host_issue_us": round(r2["host_issue_ms"] * 1e3, 2), "traffic": t_bytes, "dram_read_over_algorithmic_read": read_ratio}
            if key == "c1" and world == 1:
                e = time_steps(dist, w2.e2e_step, 10, 3)
                entry["e2e_gbps"] = round(w2.global_algorithmic_bytes() / (e["ms"] * 1e-3) / 1e9, 2)
                cpu = c1_cpu_reference(w2.global_lead)
                if cpu:
                    entry["cpu_baseline"] = cpu
            finish(key, cls, w2, entry)
            per_config[w2.name] = entry
            del w2
            torch.cuda.empty_cache()
            if world > 1:
                t1 = one_gpu_time(dist, cls, steps, 5, 1.0)
                entry["one_gpu_us"], entry["speedup"] = round(t1, 3), round(t1 / entry["us"], 3)
        except Exception as exc:  # a configuration that cannot run must not hide the headline number
            per_config[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            if world > 1:
                raise
    line["all_configs"] = detail
    if world > 1:
        bad = {k: v for k, v in checks.items() if v != "ok"}
        line["multi_gpu_check"] = "ok" if not bad else bad
        if bad:
            if dist.rank == 0:
                sys.stderr.write(json.dumps(line) + "\n")
            raise SystemExit(f"multi-GPU results differ from the oracle of the global problem: {bad}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations, the end-to-end leg, the baselines and the result check")
    ap.add_argument("--scale", type=float, default=1.0, help="fraction of the workload's leading dimension (smaller cases for profiler captures only)")
    ap.add_argument("--e2e-chunks", type=int, default=0, help="row chunks of the end-to-end leg of configuration 2 (comparison runs; 0 = the default)")
    ap.add_argument("--row-program", default="", help="row-program layout fields, e.g. copy_warpgroup=-1,ring_buffers=4 (comparison runs)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.e2e_chunks > 0:
        C2FusedExpr.E2E_CHUNKS = args.e2e_chunks
    if args.row_program:
        global ROW_PROGRAM
        ROW_PROGRAM = {k: int(v) for k, v in (kv.split("=") for kv in args.row_program.split(","))}
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch

    # stdout carries the one JSON line and nothing else: whatever libraries print (NCCL's version banner) goes to stderr
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    dist = Dist(args.gpus)
    world = dist.world
    peak, peak_kind = measured_peak()
    traffic = load_traffic()
    sampler = ClockSampler(dist.local_rank if dist.enabled else 0) if dist.rank == 0 else None
    wl, r = measure(dist, WORKLOADS[args.workload], args.steps, args.warmup, args.scale, True, sampler)
    r["steps"] = args.steps
    ms = r["ms"]
    global_bytes = wl.global_algorithmic_bytes()
    value = global_bytes / (ms * 1e-3) / 1e9
    per_gpu_gbs = wl.algorithmic_bytes() / (ms * 1e-3) / 1e9
    sus = r["sustained"]
    traffic_bytes, read_ratio = traffic_of(traffic, wl)
    kernel_launches = max(1, wl.launches_per_step)
    line = {
        "metric": "fused_expr_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "description": wl.description, "sharding": wl.sharding(),
                   "cache": f"{len(wl.sets) or 1} rotating buffer sets, {wl.algorithmic_bytes() * max(1, len(wl.sets)) >> 20} MiB on this GPU, more than 4 x L2",
                   "kernel": getattr(wl, "kernel_kind", None), "scale": args.scale},
        "elements_per_s": wl.global_units() / (ms * 1e-3),
        "host_issue_ms_per_step": r["host_issue_ms"],
        "clocks": r["clocks"],
        "gpu_launches": r["launches"],
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": traffic_bytes, "dram_read_over_algorithmic_read": read_ratio, "peak_source": f"of {peak_kind}",
                     "frac_of_nominal_8_tbs": per_gpu_gbs / 8000.0,
                     "algorithmic_bytes_per_launch": wl.algorithmic_bytes(), "launch_us": ms * 1e3 / kernel_launches,
                     "frac_sustained": wl.algorithmic_bytes() / (sus["ms_median"] * 1e-3) / 1e9 / peak,
                     "sustained": {"us_median": sus["ms_median"] * 1e3, "us_p10": sus["ms_p10"] * 1e3, "us_p90": sus["ms_p90"] * 1e3, "groups": sus["groups"],
                                   "steps_per_group": sus["steps_per_group"], "sm_mhz": (r["clocks"] or {}).get("sm_mhz")},
                     "per_config": {}},
    }
    per_config = line["roofline"]["per_config"]
    per_config[wl.name] = config_entry(wl, r, peak, world)

    if not args.no_extras:
        extras(args, dist, wl, line, per_config, peak, traffic)
    if dist.rank == 0:
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()
    dist.close()


if __name__ == "__main__":
    main()
