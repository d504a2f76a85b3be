"""The CG vector kernels (``csrc/km_cg.cu``) against their PyTorch stand-in on the same device
buffers, one step at a time, including the halo layout of a middle rank of three (emulated on one
GPU: the buffers a neighbour would have sent are filled by hand), and the row-sharded solve on two
GPUs when the box has them.

Tolerance: the kernels and the stand-in add the same numbers in a different order (fp32 partial
per row block, fp64 above), so vectors agree to 1e-6 relative and sums to 1e-5.
"""
import os

import pytest
import torch

from cg_vector_ops import TorchVectorOps

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    a, b = a.double(), b.double()
    return float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-30)


@pytest.mark.parametrize("k", [1, 3, 8, 12, 16, 40])
@pytest.mark.parametrize("layout", ["single", "halo_middle", "halo_last_ragged"])
def test_vector_kernels_match_the_stand_in(k, layout):
    from kernel_matmul_b200.cg import CudaVectorOps

    dev = torch.device("cuda:0")
    n = 128 * 23 + 57  # ragged last row block
    if layout == "single":
        row0, row1, lo, hi = 0, n, 0, n
    elif layout == "halo_middle":
        row0, row1, lo, hi = 128 * 6, 128 * 14, 128 * 4, 128 * 17
    else:
        row0, row1, lo, hi = 128 * 14, n, 128 * 11, n
    cnt = -(-(row1 - row0) // 128)
    slots, ranks = 4, 3
    seg_blocks = -(-cnt // slots) if cnt > 3 * slots else 3  # at most `slots` segments per rank
    below, above = row0 - lo, hi - row1
    top_rows, bottom_rows = 128 * 3, 128 * 3
    C, T = CudaVectorOps(dev), TorchVectorOps()

    def fresh():
        g = torch.Generator().manual_seed(k * 100 + len(layout))
        mk = lambda *s: torch.randn(*s, generator=g).to(dev)  # noqa: E731
        seg_bytes = -(-slots * k * 8 // 256) * 256
        top_off = seg_bytes
        bottom_off = top_off + -(-top_rows * k * 4 // 256) * 256
        packed = bottom_off + -(-bottom_rows * k * 4 // 256) * 256
        st = dict(x=mk(n, k), r=mk(n, k), p=mk(n, k), kp=mk(n, k), bp=torch.zeros(cnt, k, device=dev),
                  send=torch.zeros(packed, dtype=torch.uint8, device=dev), g1=torch.zeros(ranks * packed, dtype=torch.uint8, device=dev),
                  g2=torch.zeros(ranks * seg_bytes, dtype=torch.uint8, device=dev), rs=torch.rand(2, k, generator=g).to(dev) + 0.5,
                  ynorm=torch.rand(k, generator=g).to(dev) + 0.5, hist=torch.zeros(k, device=dev),
                  alpha=torch.zeros(k, device=dev), beta=torch.zeros(k, device=dev))
        # what the three ranks would have gathered: segment sums (positive) and halo rows of q
        for rk in range(ranks):
            seg = torch.rand(slots, k, generator=g, dtype=torch.float64) + 0.1
            st["g1"][rk * packed: rk * packed + slots * k * 8] = seg.to(dev).view(-1).view(torch.uint8)
            seg2 = torch.rand(slots, k, generator=g, dtype=torch.float64) + 0.1
            st["g2"][rk * seg_bytes: rk * seg_bytes + slots * k * 8] = seg2.to(dev).view(-1).view(torch.uint8)
            halo = torch.randn(top_rows + bottom_rows, k, generator=g)
            st["g1"][rk * packed + top_off: rk * packed + top_off + top_rows * k * 4] = halo[:top_rows].to(dev).view(-1).view(torch.uint8)
            st["g1"][rk * packed + bottom_off: rk * packed + bottom_off + bottom_rows * k * 4] = \
                halo[top_rows:].to(dev).view(-1).view(torch.uint8)
        st.update(seg_bytes=seg_bytes, top_off=top_off, bottom_off=bottom_off, packed=packed)
        return st

    a, b = fresh(), fresh()
    for V, st in ((C, a), (T, b)):
        # q = K p + sigma^2 p, partials of p . q, halo copies; segment sums
        V.q_dots(st["kp"], st["p"], 0.37, row0, row1, st["bp"], st["send"], st["top_off"], min(top_rows, row1 - row0),
                 st["bottom_off"], min(bottom_rows, row1 - row0))
        V.segment_sums(k, st["bp"], cnt, seg_blocks, st["send"], 0)
    torch.cuda.synchronize()
    assert _close(a["kp"], b["kp"], 1e-6)
    assert _close(a["bp"], b["bp"], 1e-5)
    segs = -(-cnt // seg_blocks)
    assert _close(a["send"][: segs * k * 8].view(torch.float64), b["send"][: segs * k * 8].view(torch.float64), 1e-5)
    tr, br = min(top_rows, row1 - row0), min(bottom_rows, row1 - row0)
    for st in (a, b):  # the halo copies are bit-exact copies of the rank's first / last rows of q
        top = st["send"][st["top_off"]: st["top_off"] + tr * k * 4].view(torch.float32).view(tr, k)
        bottom = st["send"][st["bottom_off"]: st["bottom_off"] + br * k * 4].view(torch.float32).view(br, k)
        assert torch.equal(top, st["kp"][row0: row0 + tr]) and torch.equal(bottom, st["kp"][row1 - br: row1])

    q_below = (a["g1"], 0 * a["packed"] + a["bottom_off"], row0 - bottom_rows) if below else (None, 0, 0)
    q_above = (a["g1"], 2 * a["packed"] + a["top_off"], row1) if above else (None, 0, 0)
    for V, st in ((C, a), (T, b)):
        qb = (st["g1"],) + q_below[1:] if below else q_below
        qa = (st["g1"],) + q_above[1:] if above else q_above
        V.update_xr(st["x"], st["r"], st["p"], st["kp"], qb, qa, row0, row1, lo, hi, st["g1"], st["packed"], ranks, slots,
                    st["rs"][0], st["bp"], st["alpha"])
        V.segment_sums(k, st["bp"], cnt, seg_blocks, st["send"], 0)
        V.update_p(st["p"], st["r"], lo, hi, st["g2"], st["seg_bytes"], ranks, slots, st["rs"][0], st["rs"][1], st["ynorm"],
                   st["hist"], st["beta"])
    torch.cuda.synchronize()
    assert _close(a["alpha"], b["alpha"], 1e-6) and _close(a["beta"], b["beta"], 1e-6)
    for name in ("x", "r", "p"):
        assert _close(a[name], b[name], 2e-6), name
        if layout != "single":  # nothing outside [lo, hi) (x: outside the own rows) is touched
            ref = fresh()[name]
            edge = (row0, row1) if name == "x" else (lo, hi)
            assert torch.equal(a[name][: edge[0]], ref[: edge[0]]) and torch.equal(a[name][edge[1]:], ref[edge[1]:])
    assert _close(a["bp"], b["bp"], 1e-5)
    assert _close(a["rs"], b["rs"], 1e-6) and _close(a["hist"], b["hist"], 1e-6)

    # plain inner product partials and the start of a solve
    for V, st in ((C, a), (T, b)):
        V.block_dots(st["r"], st["p"], row0, row1, st["bp"])
        V.init_scalars(k, st["g2"], st["seg_bytes"], ranks, slots, st["rs"][0], st["ynorm"])
    torch.cuda.synchronize()
    assert _close(a["bp"], b["bp"], 1e-5)
    assert _close(a["rs"][0], b["rs"][0], 1e-6) and _close(a["ynorm"], b["ynorm"], 1e-6)


def test_cg_entry_points_validate_their_arguments():
    from kernel_matmul_b200._lib import lib

    x = torch.zeros(256, 4, device="cuda")
    p = lambda t: t.data_ptr()  # noqa: E731
    assert lib.km_cg_block_dots_f32(4, p(x), p(x), 64, 256, p(x), None) == 1  # window must start at a row block
    assert b"row-block boundary" in lib.km_last_error()
    assert lib.km_cg_q_dots_f32(4, p(x), p(x), 0.1, 0, 128, p(x), None, 300, None, 0, None) == 1
    assert lib.km_cg_update_p_f32(4, p(x), p(x), 0, 256, p(x), 64, 1, 1, p(x), p(x), p(x), None, None, None) == 1
    assert b"must differ" in lib.km_last_error()


def _solve_worker(rank, world, port, out_dir, mode):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from kernel_matmul_b200 import ranges
        from kernel_matmul_b200.cg import ShardedOperator, conjugate_gradient

        torch.manual_seed(0)
        n, k, B = 40000, 8, 16
        x = torch.sort(torch.rand(n) * 1000)[0]
        params = torch.stack([torch.full((B,), 1.5), torch.rand(B), torch.full((B,), 1.0 / B)], dim=-1)
        params[0, 1] = 0.0
        y = torch.randn(n, k)
        xd = x.to(dev)
        start, end = ranges.make_ranges(6.0, xd)
        op = ShardedOperator.from_kernel("spectral", xd, params.to(dev), start, end, 0.01, mode=mode)
        res = conjugate_gradient(op, y.to(dev), iterations=30)
        torch.cuda.synchronize()
        torch.save({"x": res.solution.cpu(), "hist": res.residual_norms.cpu(), "mode": op.mode, "range": (op.lo, op.hi)},
                   os.path.join(out_dir, f"{mode}_rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_solve_equals_the_single_gpu_solve(tmp_path):
    """Rows sharded over two GPUs, halo exchange and all-gather exchange: both give the iterates of
    the single-GPU solve bit for bit (same row products, rank-count independent inner products)."""
    import torch.multiprocessing as mp

    from kernel_matmul_b200 import ranges
    from kernel_matmul_b200.cg import ShardedOperator, conjugate_gradient

    for i, mode in enumerate(("halo", "allgather")):
        mp.spawn(_solve_worker, args=(2, 29700 + (os.getpid() % 1000) + i, str(tmp_path), mode), nprocs=2, join=True)
    torch.manual_seed(0)
    n, k, B = 40000, 8, 16
    x = torch.sort(torch.rand(n) * 1000)[0]
    params = torch.stack([torch.full((B,), 1.5), torch.rand(B), torch.full((B,), 1.0 / B)], dim=-1)
    params[0, 1] = 0.0
    y = torch.randn(n, k)
    xd = x.cuda()
    start, end = ranges.make_ranges(6.0, xd)
    single = conjugate_gradient(ShardedOperator.from_kernel("spectral", xd, params.cuda(), start, end, 0.01), y.cuda(), 30)
    for mode in ("halo", "allgather"):
        for rank in range(2):
            o = torch.load(os.path.join(tmp_path, f"{mode}_rank{rank}.pt"))
            assert o["mode"] == mode
            assert torch.equal(o["x"], single.solution.cpu()), (mode, rank)
            assert torch.equal(o["hist"], single.residual_norms.cpu()), (mode, rank)
            if mode == "halo":
                assert o["range"][1] - o["range"][0] < n
