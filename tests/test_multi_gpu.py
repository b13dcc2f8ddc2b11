"""Multi-rank index logic on CPU: nnz-balanced z-slabs, halo plans and the halo exchange over gloo
(world size 2 and 3), checked against a single-process product of the same matrix.  The fused CUDA
launch itself is covered by the GPU tests; here the local product is a plain torch CSR matvec."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flexspmv_b200 import multi_gpu, problems
from oracle import ir_eval


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _local_matvec(ro, cols, vals, x_local):
    rows = ro.numel() - 1
    rid = torch.repeat_interleave(torch.arange(rows), ro[1:] - ro[:-1])
    y = torch.zeros(rows, dtype=vals.dtype)
    y.index_add_(0, rid, vals * x_local[cols.long()])
    return y


def _worker(rank, world, port, n, iters, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n2 = n * n
        bounds = multi_gpu.poisson3d_slab_bounds(n, world, "cpu")
        first_row = [b * n2 for b in bounds]
        min_col = [max(0, first_row[r] - n2) if first_row[r + 1] > first_row[r] else first_row[r] for r in range(world)]
        max_col = [min(n ** 3, first_row[r + 1] + n2) - 1 if first_row[r + 1] > first_row[r] else first_row[r] - 1
                   for r in range(world)]
        plan = multi_gpu.make_halo_plans(first_row, min_col, max_col)[rank]
        ro, cols, vals = multi_gpu.poisson3d_planes_device(n, bounds[rank], bounds[rank + 1], "cpu", col_shift=plan.col_shift)
        x_full = torch.from_numpy(problems.poisson3d(n).values["x"])
        buf = [torch.zeros(plan.local_len, dtype=torch.float64) for _ in range(2)]
        buf[0][plan.halo_lo:plan.halo_lo + plan.rows] = x_full[plan.row_begin:plan.row_end]
        cur = 0
        for _ in range(iters):
            multi_gpu.exchange_halos(buf[cur], plan)
            y = _local_matvec(ro, cols, vals, buf[cur])
            buf[1 - cur][plan.halo_lo:plan.halo_lo + plan.rows] = y
            cur = 1 - cur
        torch.save({"rows": (plan.row_begin, plan.row_end), "y": buf[cur][plan.halo_lo:plan.halo_lo + plan.rows].clone()},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_iteration_matches_single_process(world, tmp_path):
    n, iters = 12, 3
    mp.spawn(_worker, args=(world, _free_port(), n, iters, str(tmp_path)), nprocs=world, join=True)
    prob = problems.poisson3d(n)
    ro = torch.from_numpy(prob.row_offsets)
    cols = torch.from_numpy(prob.indices["selector"])
    vals = torch.from_numpy(prob.values["vals"])
    x = torch.from_numpy(prob.values["x"])
    for _ in range(iters):
        x = _local_matvec(ro, cols, vals, x)
    got = torch.zeros_like(x)
    covered = 0
    for r in range(world):
        d = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        b, e = d["rows"]
        got[b:e] = d["y"]
        covered += e - b
    assert covered == n ** 3
    assert torch.equal(got, x)       # same per-row term order on every rank: bit-identical


def test_slab_bounds_and_row_blocks_agree_with_oracle():
    n = 16
    prob = problems.poisson3d(n)
    for world in (1, 2, 3, 4, 8):
        b = multi_gpu.poisson3d_slab_bounds(n, world, "cpu")
        o = ir_eval.nnz_balanced_row_blocks(prob.row_offsets, world, n * n) // (n * n)
        assert b == o.tolist()
    ro = torch.from_numpy(problems.random_cut_csr(5000, 99999, np.random.default_rng(3)).astype(np.int64))
    for parts, snap in ((2, 1), (8, 1), (8, 64), (5, 1000)):
        mine = multi_gpu.balanced_row_blocks(ro, parts, snap)
        assert np.array_equal(mine.numpy(), ir_eval.nnz_balanced_row_blocks(ro.numpy(), parts, snap))


def test_halo_plans():
    n2 = 64
    first = [0, 4 * n2, 8 * n2, 12 * n2]
    plans = multi_gpu.make_halo_plans(first, [0, 3 * n2, 7 * n2], [5 * n2 - 1, 9 * n2 - 1, 12 * n2 - 1])
    assert [(p.halo_lo, p.halo_hi, p.send_lo, p.send_hi) for p in plans] == [(0, n2, 0, n2), (n2, n2, n2, n2), (n2, 0, n2, 0)]
    assert plans[1].col_shift == 3 * n2 and plans[1].local_len == 6 * n2
    with pytest.raises(NotImplementedError):                      # halo wider than the neighbouring block
        multi_gpu.make_halo_plans([0, 10, 12, 40], [0, 0, 0], [11, 39, 39])


def test_device_builder_matches_numpy_generator():
    n = 9
    q = problems.poisson3d(n, z_begin=2, z_end=7)
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, 2, 7, "cpu", chunk_planes=2)
    assert np.array_equal(ro.numpy(), q.row_offsets) and np.array_equal(cols.numpy(), q.indices["selector"])
    assert np.array_equal(vals.numpy(), q.values["vals"])
    assert np.array_equal(multi_gpu.poisson3d_row_offsets(n, "cpu").numpy(), problems.poisson3d(n).row_offsets)


def test_boundary_rows_and_sub_csr():
    """The rows that read a halo are exactly the first / last z-plane of an interior slab; the three
    sub-matrices tile the block and reproduce its product."""
    n, n2 = 8, 64
    first = [0, 3 * n2, 6 * n2, 8 * n2]
    plans = multi_gpu.make_halo_plans(first, [0, 2 * n2, 5 * n2], [4 * n2 - 1, 7 * n2 - 1, 8 * n2 - 1])
    x_full = torch.from_numpy(problems.poisson3d(n).values["x"])
    for plan, (z0, z1) in zip(plans, ((0, 3), (3, 6), (6, 8))):
        ro, cols, vals = multi_gpu.poisson3d_planes_device(n, z0, z1, "cpu", col_shift=plan.col_shift)
        lo, hi = multi_gpu.boundary_rows(ro, cols, plan)
        assert (lo, hi) == (n2 if plan.halo_lo else 0, n2 if plan.halo_hi else 0)
        x_local = x_full[plan.col_shift:plan.col_shift + plan.local_len]
        whole = _local_matvec(ro, cols, vals, x_local)
        got = torch.empty_like(whole)
        for r0, r1 in ((lo, plan.rows - hi), (0, lo), (plan.rows - hi, plan.rows)):
            if r1 > r0:
                sro, scols, svals = multi_gpu.sub_csr(ro, cols, vals, r0, r1)
                assert int(sro[0]) == 0 and int(sro[-1]) == scols.numel()
                got[r0:r1] = _local_matvec(sro, scols, svals, x_local)
        assert torch.equal(got, whole)
