"""world_size-2 CPU (gloo) test of the multi-GPU glue: shard ranges and the allreduce of per-rank partials.
Every rank computes the oracle statistics of its own shard; combined they must equal the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from thor_b200.sharding import combine_partials, from_ordered_keys, ordered_keys, shard_range


def test_shard_ranges_cover_and_align():
    for n in (1, 7, 8, 1000, 1 << 24, (1 << 24) + 5):
        for world in (1, 2, 3, 4, 8):
            ranges = [shard_range(n, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
                assert a1 == b0 and (a1 % 8 == 0 or a1 == n)
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) < 16  # one block of 8 plus the ragged last block


def test_ordered_keys_keep_the_float_order_and_let_nan_win():
    v = torch.tensor([float("-inf"), -3.5, -0.0, 0.0, 1e-40, 2.0, float("inf")], dtype=torch.float32)
    for high in (True, False):
        keys = ordered_keys(v, high)
        assert torch.all(keys[1:] >= keys[:-1]) and keys[1] < keys[2] and keys[4] < keys[5]
        assert torch.equal(from_ordered_keys(keys).view(torch.int32), v.view(torch.int32))
    nan = torch.tensor([float("nan"), -float("nan")], dtype=torch.float32)
    assert torch.all(ordered_keys(nan, True) > ordered_keys(v, True).max()) and torch.all(ordered_keys(nan, False) < ordered_keys(v, False).min())
    assert torch.isnan(from_ordered_keys(ordered_keys(nan, True))).all() and torch.isnan(from_ordered_keys(ordered_keys(nan, False))).all()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, rows, cols, out_path):
    import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)
    x = oracle.cast((rng.standard_normal(n) + 0.01).astype(np.float32), oracle.FP32, oracle.BF16)
    lo, hi = shard_range(n, rank, world)
    s, q, m = oracle.c4_stats(x[lo:hi], threads=1)
    sums = torch.tensor([s, q], dtype=torch.float64)
    mx = torch.tensor([m], dtype=torch.float32)
    # LayerNorm column sums over a row shard
    xs = oracle.cast(rng.standard_normal(rows * cols).astype(np.float32), oracle.FP32, oracle.BF16).reshape(rows, cols)
    dy = oracle.cast((rng.standard_normal(rows * cols) * 1e-2).astype(np.float32), oracle.FP32, oracle.BF16).reshape(rows, cols)
    gamma = oracle.cast(rng.uniform(0.9, 1.1, cols).astype(np.float32), oracle.FP32, oracle.BF16)
    r0, r1 = shard_range(rows, rank, world, multiple=1)
    _, dg, db = oracle.layernorm_bwd(xs[r0:r1], gamma, dy[r0:r1], threads=1)
    cols_sum = torch.from_numpy(np.concatenate([dg, db]))
    combine_partials(sums=sums, maxima=mx)
    combine_partials(sums=cols_sum)
    # a NaN in exactly one rank's shard is the global maximum and minimum, as in the single-GPU reductions
    nan_mx = torch.tensor([float("nan") if rank == 1 else 5.0, float(rank)], dtype=torch.float32)
    nan_mn = torch.tensor([float("nan") if rank == 0 else -5.0, float(rank)], dtype=torch.float32)
    combine_partials(maxima=nan_mx, minima=nan_mn)
    nan_ok = bool(torch.isnan(nan_mx[0]) and nan_mx[1] == world - 1 and torch.isnan(nan_mn[0]) and nan_mn[1] == 0)
    if rank == 0:
        s_all, q_all, m_all = oracle.c4_stats(x, threads=1)
        _, dg_all, db_all = oracle.layernorm_bwd(xs, gamma, dy, threads=1)
        ok = (abs(sums[0].item() - s_all) <= 1e-9 * abs(s_all) + 1e-6 and abs(sums[1].item() - q_all) <= 1e-9 * q_all and mx.item() == m_all
              and np.allclose(cols_sum.numpy(), np.concatenate([dg_all, db_all]), rtol=1e-9, atol=1e-12))
        open(out_path, "w").write("ok" if ok and nan_ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_partials_combine_across_two_ranks(tmp_path):
    out = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), 100003, 37, 256, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
