"""Flat scatter-add without atomics against the sequential loop of its definition
(Utilities/Expression/FlatScatterAddKernel.h:16-30): output[:] = 0, then output[dst] += update for every valid
destination in the order of the updates.  The first two cases are the reference's own
(test/Utilities/Expression/FlatScatterAddKernelTest.cpp:83-116, same values).  The comparison is bit for bit: the
kernels add a destination's updates in their original order, so even sums that cancel must agree with the loop."""
import numpy as np
import pytest
import torch

from thor_b200 import ThorB200InvalidArgument
from thor_b200.reductions import FlatScatterAdd, FlatScatterAddIndexPolicy as Policy, scatter_add_workspace_bytes

pytestmark = pytest.mark.gpu
SENTINEL = 0xFFFFFFFF


def _sequential(updates: np.ndarray, indices: np.ndarray, out_n: int) -> np.ndarray:
    """The definition, in float32, one update after another (np.add.at is unbuffered and in order)."""
    out = np.zeros(out_n, np.float32)
    valid = (indices != SENTINEL) & (indices.astype(np.uint64) < out_n)
    np.add.at(out, indices[valid].astype(np.int64), updates[valid])
    return out


def _run(updates, indices, out_n, policy=Policy.CanonicalizeDuplicatesAndSkipInvalid, fill=9.0):
    u = torch.from_numpy(np.asarray(updates, np.float32)).cuda()
    i = torch.from_numpy(np.asarray(indices, np.uint32)).cuda()
    out = torch.full((out_n,), fill, device="cuda")
    plan = FlatScatterAdd(u, i, out, policy)
    plan.run(u, i, out)
    torch.cuda.synchronize()
    return plan, out.cpu().numpy()


def test_unique_valid_indices_use_the_direct_path():
    plan, got = _run([1.5, -2.0, 3.0], [4, 0, 2], 6, Policy.IndicesAreUniqueAndValid)
    assert plan.index_policy == Policy.IndicesAreUniqueAndValid and plan.workspace_bytes == 0 and plan.kernel_launches == 1
    assert got.tolist() == [-2.0, 0.0, 3.0, 0.0, 1.5, 0.0]


def test_canonicalized_path_sums_duplicates_and_skips_invalid_indices():
    plan, got = _run([1.0, 2.0, 3.0, 4.0, 5.0], [2, SENTINEL, 2, 6, 0], 5)
    assert plan.index_policy == Policy.CanonicalizeDuplicatesAndSkipInvalid and plan.workspace_bytes > 0
    assert got.tolist() == [5.0, 0.0, 4.0, 0.0, 0.0]


@pytest.mark.parametrize("n,out_n,invalid", [(1, 1, 0.0), (31, 7, 0.2), (4096, 255, 0.0), (4097, 256, 0.1), (100_000, 1000, 0.05), (1 << 20, 70_000, 0.01),
                                             (300_001, (1 << 24) + 5, 0.3), (1 << 22, 1 << 22, 0.0)])
def test_random_destinations_match_the_sequential_loop_bit_for_bit(n, out_n, invalid):
    rng = np.random.default_rng(n * 31 + out_n)
    updates = (rng.standard_normal(n) * 10.0 ** rng.integers(-3, 4, n)).astype(np.float32)  # mixed magnitudes: the order of a sum matters
    indices = rng.integers(0, out_n, n, dtype=np.uint64).astype(np.uint32)
    bad = rng.random(n) < invalid
    indices[bad] = np.where(rng.random(int(bad.sum())) < 0.5, SENTINEL, np.minimum(out_n + rng.integers(0, 1000, int(bad.sum())), SENTINEL - 1)).astype(np.uint32)
    plan, got = _run(updates, indices, out_n)
    want = _sequential(updates, indices, out_n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    passes = max(1, (int(out_n - 1).bit_length() + 7) // 8)
    assert plan.kernel_launches == 3 * passes + 1


def test_every_small_size_with_many_and_few_duplicates():
    """Sizes around the chunk of eight pairs a thread walks and the 256 pairs of a warp's window, with three destinations
    (runs span threads and warps) and with fifty (most runs inside one thread)."""
    rng = np.random.default_rng(77)
    for n in list(range(1, 41)) + [63, 64, 65, 255, 256, 257, 258, 511, 512, 513, 2047, 2048, 2049]:
        for out_n in (3, 50):
            updates = (rng.standard_normal(n) * 10.0 ** rng.integers(-3, 4, n)).astype(np.float32)
            indices = rng.integers(0, out_n + 1, n).astype(np.uint32)  # out_n itself is out of range: skipped
            _, got = _run(updates, indices, out_n)
            assert np.array_equal(got.view(np.uint32), _sequential(updates, indices, out_n).view(np.uint32)), (n, out_n)


def test_long_runs_of_one_destination_keep_the_order_of_the_updates():
    """Running-maximum positions repeat for long stretches: runs far longer than a warp, some of them crossing the
    tiles of the sort, plus one destination that collects a third of all updates."""
    rng = np.random.default_rng(5)
    n, out_n = 200_000, 5000
    run_starts = np.sort(rng.choice(n, 300, replace=False))
    indices = np.zeros(n, np.uint32)
    dest = rng.integers(0, out_n, run_starts.size + 1)
    indices[:] = dest[np.searchsorted(run_starts, np.arange(n), side="right")]
    indices[rng.random(n) < 0.33] = 4999
    updates = (rng.standard_normal(n) * 10.0 ** rng.integers(-4, 5, n)).astype(np.float32)
    _, got = _run(updates, indices, out_n)
    assert np.array_equal(got.view(np.uint32), _sequential(updates, indices, out_n).view(np.uint32))


def test_negative_zero_updates_and_all_invalid_inputs():
    _, got = _run([-0.0, -0.0, 1.0], [1, 1, SENTINEL], 3)
    assert got.view(np.uint32).tolist() == [0, 0, 0], "+0 + -0 is +0, as in the loop that starts from a zero-filled output"
    _, got = _run([1.0, 2.0], [SENTINEL, 7], 4)
    assert got.tolist() == [0.0] * 4
    _, got = _run(np.zeros(0, np.float32), np.zeros(0, np.uint32), 4)
    assert got.tolist() == [0.0] * 4, "no updates: the output is only cleared"


def test_results_are_identical_on_every_run_and_the_plan_is_reusable():
    rng = np.random.default_rng(9)
    n, out_n = 500_000, 3000
    u = torch.from_numpy((rng.standard_normal(n) * 1e3).astype(np.float32)).cuda()
    i = torch.from_numpy(rng.integers(0, out_n, n).astype(np.uint32)).cuda()
    out = torch.empty(out_n, device="cuda")
    plan = FlatScatterAdd(u, i, out)
    first = plan.run(u, i, out).clone()
    for _ in range(5):
        assert torch.equal(plan.run(u, i, out).view(torch.int32), first.view(torch.int32))
    u2 = u.flip(0).contiguous()
    plan.run(u2, i, out)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), _sequential(u2.cpu().numpy(), i.cpu().numpy(), out_n).view(np.uint32))


def test_misuse_is_rejected_like_the_reference():
    u, i, out = torch.zeros(4, device="cuda"), torch.zeros(4, device="cuda", dtype=torch.uint32), torch.zeros(8, device="cuda")
    with pytest.raises(ThorB200InvalidArgument, match="UINT32"):
        FlatScatterAdd(u, i.to(torch.int32), out)
    with pytest.raises(ThorB200InvalidArgument, match="same dtype"):
        FlatScatterAdd(u, i, out.half())
    with pytest.raises(ThorB200InvalidArgument, match="same shape"):
        FlatScatterAdd(u, i[:3], out)
    with pytest.raises(ThorB200InvalidArgument, match="only fp32"):
        FlatScatterAdd(u.half(), i, out.half())
    plan = FlatScatterAdd(u, i, out)
    with pytest.raises(ThorB200InvalidArgument, match="do not match the prepared plan"):
        plan.run(u[:2], i[:2], out)
    assert scatter_add_workspace_bytes(0, 10) == 1
