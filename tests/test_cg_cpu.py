"""Host logic of the row-sharded CG solve on CPU: world_size-2 gloo ranks against a single
process and against a dense fp64 solve.  The matvec is a dense torch product here (the CUDA
kernel needs a GPU); sharding, the all-gathers, the row-sharded vector updates and the
block-ordered inner products are the code under test."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernel_matmul_b200.cg import ShardedOperator, conjugate_gradient, row_block_window


def _system(n=700, k=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.sort(torch.rand(n, generator=g) * 30)[0].double()
    K = torch.exp(-0.5 * (x[:, None] - x[None, :]) ** 2 / 0.8**2) * torch.cos(2 * torch.pi * 0.3 * (x[:, None] - x[None, :]))
    K = K * ((x[:, None] - x[None, :]).abs() <= 4.0)  # banded, symmetric
    y = torch.randn(n, k, generator=g, dtype=torch.float64)
    return K, y


def _dense_matvec(K):
    def matvec_rows(v, rb_begin, rb_count, out):
        r0 = rb_begin * 128
        out.copy_(K[r0 : r0 + out.shape[0]] @ v)

    return matvec_rows


def test_row_block_windows_cover_everything():
    for R in (1, 5, 8, 33):
        for world in (1, 2, 3, 8):
            wins = [row_block_window(R, r, world) for r in range(world)]
            covered = []
            for b, c in wins:
                covered += list(range(b, b + c))
            assert covered == list(range(R))
            assert len({b for b, _ in wins if _ > 0}) == len([1 for _, c in wins if c > 0])


def test_cg_single_process_matches_dense_solve():
    K, y = _system()
    op = ShardedOperator(K.shape[0], 0.05, _dense_matvec(K))
    res = conjugate_gradient(op, y, iterations=200, tol=1e-12)
    ref = torch.linalg.solve(K + 0.05 * torch.eye(K.shape[0], dtype=torch.float64), y)
    assert float((res.solution - ref).abs().max() / ref.abs().max()) < 1e-8
    assert res.residual_norms.shape[1] == y.shape[1]
    assert bool((res.residual_norms[-1] < 1e-10).all())


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        K, y = _system()
        op = ShardedOperator(K.shape[0], 0.05, _dense_matvec(K))
        assert (op.rank, op.world) == (rank, world)
        res = conjugate_gradient(op, y, iterations=25)
        torch.save({"x": res.solution, "hist": res.residual_norms, "window": (op.begin, op.count)},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_cg_sharded_ranks_agree_with_single_process(tmp_path, world):
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    K, y = _system()
    single = conjugate_gradient(ShardedOperator(K.shape[0], 0.05, _dense_matvec(K)), y, iterations=25)
    outs = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    windows = [o["window"] for o in outs]
    assert sum(c for _, c in windows) == -(-K.shape[0] // 128)
    for o in outs:
        # identical iterates on every rank and for every rank count (same row products, inner
        # products added per row block and then in block order)
        assert torch.equal(o["x"], single.solution)
        assert torch.equal(o["hist"], single.residual_norms)
