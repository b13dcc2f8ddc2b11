"""Two ranks on two GPUs (NCCL): the partitioned iteration x <- A x against the same iteration on one GPU.
Skipped when fewer than two devices are visible."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, iters, overlap, out_dir, graph=False):
    import torch.distributed as dist
    from flexspmv_b200 import multi_gpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n2 = n * n
    bounds = multi_gpu.poisson3d_slab_bounds(n, world, dev)
    first_row = [b * n2 for b in bounds]
    min_col = [max(0, first_row[r] - n2) for r in range(world)]
    max_col = [min(n ** 3, first_row[r + 1] + n2) - 1 for r in range(world)]
    plan = multi_gpu.make_halo_plans(first_row, min_col, max_col)[rank]
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, bounds[rank], bounds[rank + 1], dev, col_shift=plan.col_shift)
    g = torch.Generator(device="cpu")
    g.manual_seed(7)
    x_full = (torch.rand(n ** 3, generator=g, dtype=torch.float64) * 2 - 1)
    op = multi_gpu.PartitionedSpmv(plan, ro, cols, vals, x_full[plan.row_begin:plan.row_end].to(dev), overlap=overlap)
    captured = None
    if graph:
        captured = op.capture_pair()          # runs one eager pair on the capture stream, then captures a pair
        for _ in range((iters - 2) // 2):
            op.step_pair()
    else:
        for _ in range(iters):
            op.step()
    torch.cuda.synchronize()
    op.ext.check()
    torch.save({"rows": (plan.row_begin, plan.row_end), "y": op.owned().cpu(), "captured": captured,
                "graph_error": op.graph_error}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    os._exit(0)      # no communicator teardown: nothing is in flight and the results are on disk


@pytest.mark.parametrize("overlap,graph", [(False, False), (True, False), (False, True), (True, True)],
                         ids=["eager", "eager-overlap", "graph", "graph-overlap"])
def test_two_ranks_match_one_gpu(overlap, graph, tmp_path):
    """Eager steps, and (graph) a captured pair of iterations replayed: the capture must succeed on both ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flexspmv_b200 import multi_gpu
    from flexspmv_b200.binding import load_builtin
    n, iters = 48, 6
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, iters, overlap, str(tmp_path), graph)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, 0, n, dev)
    g = torch.Generator(device="cpu")
    g.manual_seed(7)
    x = (torch.rand(n ** 3, generator=g, dtype=torch.float64) * 2 - 1).to(dev)
    ext = load_builtin("spmv")
    for _ in range(iters):
        y = torch.empty_like(x)
        ext.launch_into([vals, x], [cols], ro, [y], n ** 3, cols.numel(), n ** 3)
        x = y
    ref = x.cpu()
    got = torch.empty_like(ref)
    for r in range(2):
        d = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        got[d["rows"][0]:d["rows"][1]] = d["y"]
        if graph:
            assert d["captured"] is True, d["graph_error"]
    # rows that straddle a CTA boundary add their two partial sums in a different association when the
    # blocks (and so the CTA boundaries) differ: agreement to the fp64 parity tolerance, not bit for bit
    scale = float(ref.abs().max())
    assert float((got - ref).abs().max()) <= 1e-12 * scale * iters


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_two_devices():
    """The library's per-device state (shared-memory opt-in of the kernels, SM count, plan cache) must not be
    tied to the first device a process used."""
    from flexspmv_b200 import graphs, problems
    from flexspmv_b200.binding import GraphExtension
    ir = graphs.spmv_graph()
    ext = GraphExtension(ir)
    prob = problems.random_problem(ir, 5000, 5000, 80000, seed=31, dtype=np.float64)
    results = []
    for d in (0, 1, 0):
        dev = torch.device("cuda", d)
        vals = torch.from_numpy(prob.values["vals"]).to(dev)
        x = torch.from_numpy(prob.values["x"]).to(dev)
        cols = torch.from_numpy(prob.indices["selector"]).to(dev)
        ro = torch.from_numpy(prob.row_offsets).to(dev)
        (y,) = ext.merged_spmv_launch(vals, x, cols, ro, prob.num_rows, prob.num_cols)
        torch.cuda.synchronize(dev)
        assert y.device == dev
        results.append(y.cpu())
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
