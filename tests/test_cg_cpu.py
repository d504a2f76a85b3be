"""Host logic of the row-sharded CG solve on CPU: world_size-2/3/8 gloo ranks against a single
process and against a dense fp64 solve.  The matvec is a dense torch product and the vector
steps are the PyTorch stand-in of ``tests/cg_vector_ops.py`` (the CUDA kernels need a GPU);
sharding by segments, the halo and all-gather exchanges, the buffer layout and the agreement
check between ranks are the code under test."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cg_vector_ops import TorchVectorOps
from kernel_matmul_b200.cg import (CGSolver, ShardedOperator, ShardMismatchError, conjugate_gradient, row_block_window,
                                   segment_layout)

CUTOFF = 4.0


def _system(n=1500, k=3, seed=0, span=30.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.sort(torch.rand(n, generator=g) * span)[0].double()
    K = torch.exp(-0.5 * (x[:, None] - x[None, :]) ** 2 / 0.8**2) * torch.cos(2 * torch.pi * 0.3 * (x[:, None] - x[None, :]))
    K = K * ((x[:, None] - x[None, :]).abs() <= CUTOFF)  # banded, symmetric
    y = torch.randn(n, k, generator=g, dtype=torch.float64)
    return x, K, y


def _col_range(x, rb_begin, rb_count):
    """Columns the rows of a window of row blocks touch (exact for the |tau| <= CUTOFF mask)."""
    n = x.shape[0]
    r0, r1 = rb_begin * 128, min(n, (rb_begin + rb_count) * 128)
    if r1 <= r0:
        return (0, 0)
    lo = int(torch.searchsorted(x, x[r0] - CUTOFF, right=False))
    hi = int(torch.searchsorted(x, x[r1 - 1] + CUTOFF, right=True))
    return lo, hi


def _dense_matvec(K, x=None):
    """Dense product of a window of row blocks.  With ``x`` every row block reads the vector only on
    the columns of its own band (as the banded kernel does; the solver keeps nothing else current
    in halo mode) -- the same arithmetic per row block whatever the window, so results can be
    compared bit for bit between rank counts."""
    def matvec_rows(v, rb_begin, rb_count, out):
        r0 = rb_begin * 128
        if x is None:
            out.copy_(K[r0: r0 + out.shape[0]] @ v)
            return
        for rb in range(rb_begin, rb_begin + rb_count):
            lo, hi = _col_range(x, rb, 1)
            rows = slice(rb * 128, min((rb + 1) * 128, K.shape[0]))
            out[rows.start - r0: rows.stop - r0] = K[rows, lo:hi] @ v[lo:hi]

    return matvec_rows


def test_segments_and_windows_cover_everything():
    for R in (1, 5, 8, 33, 64, 65, 1000, 32768):
        for world in (1, 2, 3, 8):
            seg_blocks, nseg, per_rank = segment_layout(R, world)
            assert nseg <= 64 and (nseg - 1) * seg_blocks < R <= nseg * seg_blocks
            wins = [row_block_window(R, r, world) for r in range(world)]
            covered = []
            for b, c in wins:
                assert c == 0 or b % seg_blocks == 0  # whole segments
                covered += list(range(b, b + c))
            assert covered == list(range(R))
    assert row_block_window(32768, 3, 8) == (3 * 4096, 4096)


def test_cg_single_process_matches_dense_solve():
    _, K, y = _system(n=700)
    op = ShardedOperator(K.shape[0], 0.05, _dense_matvec(K), vector_ops=TorchVectorOps())
    assert op.mode == "single"
    res = conjugate_gradient(op, y, iterations=200, tol=1e-12)
    ref = torch.linalg.solve(K + 0.05 * torch.eye(K.shape[0], dtype=torch.float64), y)
    assert float((res.solution - ref).abs().max() / ref.abs().max()) < 1e-8
    assert res.residual_norms.shape[1] == y.shape[1]
    assert bool((res.residual_norms[-1] < 1e-10).all())
    assert res.iterations < 200


def test_solver_refuses_cpu_tensors_without_a_stand_in():
    _, K, y = _system(n=300)
    op = ShardedOperator(K.shape[0], 0.05, _dense_matvec(K))
    with pytest.raises(RuntimeError, match="no CPU path"):
        CGSolver(op, y)


def _worker(rank, world, port, out_dir, mode, n, span):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, K, y = _system(n=n, span=span)
        R = -(-n // 128)
        begin, count = row_block_window(R, rank, world)
        if mode == "halo":
            cr = _col_range(x, begin, count)
            lo_blk = (cr[0] // 128) * 128
            hi_blk = min(n, -(-cr[1] // 128) * 128)
            columns = (min(lo_blk, begin * 128), max(hi_blk, min(n, (begin + count) * 128)))
            op = ShardedOperator(n, 0.05, _dense_matvec(K, x), col_range=cr, vector_ops=TorchVectorOps(), mode="auto")
            assert (op.lo, op.hi) == columns
        else:
            op = ShardedOperator(n, 0.05, _dense_matvec(K, x), vector_ops=TorchVectorOps(), mode=mode)
        assert (op.rank, op.world) == (rank, world)
        res = conjugate_gradient(op, y, iterations=25)
        torch.save({"x": res.solution, "hist": res.residual_norms, "window": (op.begin, op.count), "mode": op.mode,
                    "range": (op.lo, op.hi)}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode,n,span", [(2, "allgather", 1500, 30.0), (3, "allgather", 1500, 30.0), (2, "halo", 3000, 30.0),
                                               (3, "halo", 4500, 30.0), (8, "halo", 5000, 64.0), (8, "allgather", 2000, 30.0)])
def test_cg_sharded_ranks_agree_with_single_process(tmp_path, world, mode, n, span):
    port = 29500 + (os.getpid() % 2000) + world + (10 if mode == "halo" else 0)
    mp.spawn(_worker, args=(world, port, str(tmp_path), mode, n, span), nprocs=world, join=True)
    x, K, y = _system(n=n, span=span)
    single = conjugate_gradient(ShardedOperator(n, 0.05, _dense_matvec(K, x), vector_ops=TorchVectorOps()), y, iterations=25)
    outs = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    assert sum(o["window"][1] for o in outs) == -(-n // 128)
    for o in outs:
        assert o["mode"] == mode
        if mode == "halo":  # a real halo: neither the own rows only nor everything
            assert o["range"][1] - o["range"][0] < n
        # identical iterates on every rank and for every rank count (same row products, inner
        # products added per row block, per segment and then in segment order)
        assert torch.equal(o["x"], single.solution)
        assert torch.equal(o["hist"], single.residual_norms)


def _mismatch_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = 1500 if rank == 0 else 1400  # rank 1 was handed another system
        _, K, _ = _system(n=n)
        try:
            ShardedOperator(n, 0.05, _dense_matvec(K), vector_ops=TorchVectorOps())
            outcome = "no error"
        except ShardMismatchError as exc:
            outcome = str(exc)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(outcome)
    finally:
        dist.destroy_process_group()


def test_ranks_that_describe_different_systems_all_raise(tmp_path):
    port = 29500 + (os.getpid() % 2000) + 50
    mp.spawn(_mismatch_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        msg = open(os.path.join(tmp_path, f"rank{rank}.txt")).read()
        assert "rank 1 describes a different system than rank 0" in msg, msg


def test_a_non_finite_residual_is_reported():
    """A product that returns NaN rows (what a tensor-core kernel that gave up writes) surfaces
    through ``check_finite`` instead of going unnoticed."""
    _, K, y = _system(n=700)

    def broken(v, rb_begin, rb_count, out):
        out.fill_(float("nan"))

    solver = CGSolver(ShardedOperator(K.shape[0], 0.05, broken, vector_ops=TorchVectorOps()), y)
    solver.step()
    with pytest.raises(RuntimeError, match="non-finite residual"):
        solver.check_finite()
    good = CGSolver(ShardedOperator(K.shape[0], 0.05, _dense_matvec(K), vector_ops=TorchVectorOps()), y)
    good.step()
    good.check_finite()
