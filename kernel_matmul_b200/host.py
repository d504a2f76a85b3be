"""Forward product and hyper-parameter gradients for operands that live in host memory.

``matmul_and_grad_from_host`` is ``ops.matmul`` followed by ``ops.matmul_bwd`` for callers whose
data sits in (pinned) host buffers: inputs are copied in on a copy stream, the kernels run on
the current stream, results are copied out on a second copy stream, and the three overlap --
the gradient's ``out_grad`` arrives while the product runs, the product's output leaves while
the gradient runs.  The reference has no counterpart (its ops take device tensors only,
native/common/entrypoint.h:3-14); this is the path ``bench.py`` times end to end.
"""
from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor

from . import ops


class HostStreams:
    """The two copy streams of a device, created once and reused."""

    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)


def matmul_and_grad_from_host(
    kernel_type: str,
    x: Tensor,
    rhs: Tensor,
    params: Tensor,
    out_grad: Tensor,
    make_band: Callable[[Tensor], tuple[Tensor, Tensor]],
    out: Tensor,
    grad: Tensor,
    streams: HostStreams,
    *,
    path: str = "auto",
) -> None:
    """``out[...] = K(x, x; params) @ rhs`` and ``grad[...] = d sum(out_grad * out) / d params``.

    ``x (n,)``, ``rhs (n, k)``, ``params (B, P)``, ``out_grad (B, n, k)`` are host tensors (pinned
    for the copies to be asynchronous); ``x`` and ``rhs`` are shared by the ``B`` kernels.
    ``make_band(x_device) -> (start, end)`` builds the band on the device.  ``out (B, n, k)`` and
    ``grad (B, P)`` are host tensors that receive the results.  All work is ordered after what is
    already queued on the current stream, and the current stream waits for the last copy: an
    event recorded on it after the call marks the completion of everything.
    """
    dev = streams.device
    cur = torch.cuda.current_stream(dev)
    B = params.shape[0]
    streams.copy_in.wait_stream(cur)
    with torch.cuda.stream(streams.copy_in):
        dx = x.to(dev, non_blocking=True)
        drhs = rhs.to(dev, non_blocking=True)
        dp = params.to(dev, non_blocking=True)
        forward_inputs = torch.cuda.Event()
        forward_inputs.record(streams.copy_in)
        dog = out_grad.to(dev, non_blocking=True)
        gradient_inputs = torch.cuda.Event()
        gradient_inputs.record(streams.copy_in)
    for t in (dx, drhs, dp, dog):
        t.record_stream(cur)

    cur.wait_event(forward_inputs)
    start, end = make_band(dx)
    dxb = dx.expand(B, -1)
    drhsb = drhs.expand(B, -1, -1)
    d_out = ops.matmul(kernel_type, dxb, dxb, drhsb, dp, start, end, path=path)
    product_done = torch.cuda.Event()
    product_done.record(cur)
    with torch.cuda.stream(streams.copy_out):
        streams.copy_out.wait_event(product_done)
        out.copy_(d_out, non_blocking=True)
    d_out.record_stream(streams.copy_out)

    cur.wait_event(gradient_inputs)
    d_grad = ops.matmul_bwd(kernel_type, dxb, dxb, drhsb, dp, start, end, dog, path=path)
    gradient_done = torch.cuda.Event()
    gradient_done.record(cur)
    with torch.cuda.stream(streams.copy_out):
        streams.copy_out.wait_event(gradient_done)
        grad.copy_(d_grad, non_blocking=True)
    d_grad.record_stream(streams.copy_out)
    cur.wait_stream(streams.copy_out)


def cg_solve_from_host(
    kernel_type: str,
    x: Tensor,
    params: Tensor,
    y: Tensor,
    cutoff: float | None,
    sigma2: float,
    iterations: int,
    out: Tensor,
    device: torch.device,
    *,
    group=None,
    mode: str = "auto",
):
    """``(sum_b K_b(x, x; params[b]) + sigma2 I) V = y`` by ``iterations`` steps of the row-sharded CG,
    for operands in (pinned) host memory.

    ``x (n,)``, ``params (B, P)`` or ``(P,)``, ``y (n, k)`` and ``out (n, k)`` are host tensors.  Every
    rank copies ``x`` and ``params`` in full (the band is built from all of ``x``) but of ``y`` only
    the rows it keeps current (its own rows plus the band's halo), runs the solve, and copies ITS
    rows of the solution into ``out[row0:row1]`` -- nothing else of ``out`` is written.  Returns
    ``(solver, (row0, row1))``; the copy out is asynchronous on the current stream.  The reference
    has no counterpart: its solves go through ``linear_operator``'s CG on device tensors
    (tests/test_linear_operator.py:38).
    """
    from . import ranges
    from .cg import CGSolver, ShardedOperator

    dx = x.to(device, non_blocking=True)
    dp = params.to(device, non_blocking=True)
    start, end = ranges.make_ranges(cutoff, dx)
    op = ShardedOperator.from_kernel(kernel_type, dx, dp, start, end, sigma2, group=group, mode=mode)
    solver = CGSolver(op, y, max_iterations=max(iterations, 1))
    for _ in range(iterations):
        solver.step()
    if op.rows > 0:
        out[op.row0: op.row1].copy_(solver.solution_rows(), non_blocking=True)
    return solver, (op.row0, op.row1)
