"""Tensor-parallel shard layout on CPU ranks (gloo, world_size 2): the split the reference's
ColumnParallelLinear / RowParallelLinear make (model.py:208-267) and bench.py reproduces.

Row-parallel: rank r holds columns [r*K/ws, (r+1)*K/ws) of W and the matching slice of x; K/ws is a multiple
of 128, so every rank's act_quant blocks and weight scale blocks are exactly the corresponding blocks of the
unsharded tensors, and the all_reduce of the partial outputs equals the full GEMM up to the bf16 rounding of
each partial.  Column-parallel: rank r holds rows [r*N/ws, ...) of W and produces that slice of the output."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 24, 256, 1024
        x, w, wq, ws = O.make_case(M, N, K, 61)
        xq, xs = O.act_quant(x)
        full = O.fp8_gemm(xq, xs, wq, ws).float()
        # ---- row-parallel (model.py:237-267): K split, partial sums all_reduced
        ks = K // world
        x_r = x[:, rank * ks:(rank + 1) * ks].contiguous()
        xq_r, xs_r = O.act_quant(x_r)
        assert torch.equal(xq_r.view(torch.uint8), xq.view(torch.uint8)[:, rank * ks:(rank + 1) * ks])
        assert torch.equal(xs_r, xs[:, rank * ks // 128:(rank + 1) * ks // 128])
        wq_r = wq.view(torch.uint8)[:, rank * ks:(rank + 1) * ks].contiguous().view(torch.float8_e4m3fn)
        ws_r = ws[:, rank * ks // 128:(rank + 1) * ks // 128].contiguous()
        part = O.fp8_gemm(xq_r, xs_r, wq_r, ws_r).float()       # bf16 partial, as RowParallelLinear produces
        dist.all_reduce(part)
        ok_row, ratio_row = O.gemm_tolerance_ok(part.to(torch.bfloat16), full.to(torch.bfloat16))
        # ---- column-parallel (model.py:208-234): N split, no communication
        ns = N // world
        wq_c = wq.view(torch.uint8)[rank * ns:(rank + 1) * ns].contiguous().view(torch.float8_e4m3fn)
        ws_c = ws[rank * ns // 128:(rank + 1) * ns // 128].contiguous()
        col = O.fp8_gemm(xq, xs, wq_c, ws_c).float()
        ok_col = torch.equal(col, full[:, rank * ns:(rank + 1) * ns])
        # ---- the benchmark's accounting: shards add up to the single-GPU problem set
        import bench
        mine = sum(bench.gemm_flops(m, n, k) for m in bench.MS for (_, k, n, _, _, c) in bench.sweep_rows(world, rank) if c)
        t = torch.tensor([mine], dtype=torch.float64)
        dist.all_reduce(t)
        ref = sum(bench.gemm_flops(m, n, k) for m in bench.MS for (_, k, n, *_r) in bench.sweep_rows(1))
        q.put((rank, ok_row, ratio_row, ok_col, abs(t.item() - ref) <= 1e-9 * ref))
    finally:
        dist.destroy_process_group()


def test_tp_shards_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_row, ratio_row, ok_col, ok_flops in res:
        assert ok_row, f"rank {rank}: row-parallel sum outside tolerance ({ratio_row:.3f})"
        assert ok_col, f"rank {rank}: column-parallel slice differs"
        assert ok_flops, f"rank {rank}: sharded flop count does not add up"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_bench_shards_add_up_to_the_single_gpu_problem_set(world):
    """bench.py --gpus N: the ranks' counted problems cover the single-GPU sweep exactly once (strong scaling),
    every shard keeps K a multiple of the 128-wide quantisation block, and row-parallel shards all_reduce."""
    sys.path.insert(0, ROOT)
    import bench
    ref = sum(bench.gemm_flops(m, n, k) for m in bench.MS for (_, k, n, *_r) in bench.sweep_rows(1))
    total = 0
    for rank in range(world):
        rows = bench.sweep_rows(world, rank)
        for name, k, n, _, all_reduce, counted in rows:
            assert k % 128 == 0 and n > 0, (world, rank, name)
            if all_reduce:
                assert f"/tp{world}" in name, name
        total += sum(bench.gemm_flops(m, n, k) for m in bench.MS for (_, k, n, _, _, c) in rows if c)
    assert abs(total - ref) <= 1e-9 * ref
