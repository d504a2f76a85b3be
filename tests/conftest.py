"""Shared test helpers.

``-m "not gpu"`` tests run without a GPU (oracle vs fixtures, host logic, library symbols);
``-m gpu`` tests are the parity tests of the CUDA path against the oracle.
"""
from __future__ import annotations

import os
import random
import sys
from dataclasses import dataclass

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_terminal_summary(terminalreporter):
    """Which clause of the gradient criterion the gradient checks passed by: per test function the
    number of compared elements, how many met the plain 1e-5 relative bound, the largest relative
    error seen and the largest error in units of the cancellation-free scale."""
    if not GRAD_STATS:
        return
    tr = terminalreporter
    tr.write_sep("-", "gradient criterion: |err| <= 1e-5 |ref|  or  |err| <= 1e-6 sum|terms|")
    tr.write_line(f"{'test':58s} {'elements':>9s} {'strict':>9s} {'max rel err':>12s} {'max err/scale':>14s}")
    for name, (count, strict, max_rel, max_scaled) in sorted(GRAD_STATS.items()):
        tr.write_line(f"{name:58s} {count:9d} {strict:9d} {max_rel:12.3e} {max_scaled:14.3e}")


@pytest.fixture(autouse=True)
def seed(request) -> int:
    rng = random.Random(request.node.nodeid)
    s = rng.randint(0, 2**31 - 1)
    random.seed(s)
    torch.manual_seed(s)
    return s


KERNEL_TYPES = ["rbf", "spectral", "locally_periodic"]

# (m, n, batch, unsqueeze, k, cutoff): the input family of the reference's native tests
# (tests/conftest.py:48-55): ragged last blocks, expanded (stride-0) batches, k = 1 / 11 / 65.
SHAPES = [
    dict(m=128, n=128, batch=(), unsqueeze=None, k=1, cutoff=2.0),
    dict(m=600, n=800, batch=(), unsqueeze=None, k=11, cutoff=2.0),
    dict(m=500, n=500, batch=(3,), unsqueeze=None, k=11, cutoff=2.0),
    dict(m=301, n=201, batch=(3,), unsqueeze=0, k=11, cutoff=None),
    dict(m=301, n=199, batch=(2, 3), unsqueeze=1, k=11, cutoff=2.0),
    dict(m=129, n=130, batch=(), unsqueeze=None, k=65, cutoff=2.0),
]


@dataclass
class Example:
    x1: torch.Tensor
    x2: torch.Tensor
    rhs: torch.Tensor
    params: torch.Tensor
    start: torch.Tensor
    end: torch.Tensor
    kernel_type: str
    cutoff: float | None

    def to(self, device):
        return Example(
            self.x1.to(device), self.x2.to(device), self.rhs.to(device), self.params.to(device),
            self.start.to(device), self.end.to(device), self.kernel_type, self.cutoff,
        )


def make_params(kernel_type: str, batch: tuple[int, ...], lengthscale_factor: float = 1.0) -> torch.Tensor:
    """theta = 1 + U[0,1) per entry (frequency 0.5 + U/2), as tests/conftest.py:116-132."""
    if kernel_type == "rbf":
        cols = [(1 + torch.rand(batch)) * lengthscale_factor, 1 + torch.rand(batch)]
    elif kernel_type == "spectral":
        cols = [(1 + torch.rand(batch)) * lengthscale_factor, 0.5 + torch.rand(batch) * 0.5, 1 + torch.rand(batch)]
    else:
        cols = [
            (1 + torch.rand(batch)) * lengthscale_factor,
            1 + torch.rand(batch) * lengthscale_factor,
            1 + torch.rand(batch),
            1 + torch.rand(batch),
        ]
    return torch.stack(cols, dim=-1).float()


def make_example(shape: dict, kernel_type: str, *, square: bool = False, align: bool = False) -> Example:
    """CPU tensors; ranges from the oracle's restatement of the reference scans."""
    from oracle import oracle as O

    m = shape["m"]
    n = shape["n"] if not square else m
    batch, unsq, k, cutoff = shape["batch"], shape["unsqueeze"], shape["k"], shape["cutoff"]
    sq_batch = batch if unsq is None else (*batch[:unsq], *batch[unsq + 1 :])
    x1 = torch.sort(torch.rand(*sq_batch, m) * 10, dim=-1)[0]
    x2 = x1 if square else torch.sort(torch.rand(*sq_batch, n) * 10, dim=-1)[0]
    if square:
        start, end = O.make_ranges(cutoff, x1, block_size=128)
    else:
        start, end = O.make_ranges(cutoff, x1, x2, block_size=128, align=align)
    rhs = torch.randn(*sq_batch, n, k)
    rhs = rhs / torch.linalg.norm(rhs, dim=-2, keepdim=True)
    if unsq is not None:
        x1 = x1.unsqueeze(unsq).expand(*batch, m)
        x2 = x2.unsqueeze(unsq).expand(*batch, n)
        start = start.unsqueeze(unsq).expand(*batch, -1)
        end = end.unsqueeze(unsq).expand(*batch, -1)
        rhs = rhs.unsqueeze(unsq).expand(*batch, n, k)
    params = make_params(kernel_type, batch)
    return Example(x1, x2, rhs, params, start, end, kernel_type, cutoff)


def rel_err(actual: torch.Tensor, expected: torch.Tensor, dim=None) -> float:
    """max |actual - expected| / max |expected| (norm-wise relative error; outputs cross zero)."""
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    denom = e.abs().max().clamp_min(1e-300)
    return float((a - e).abs().max() / denom)


GRAD_RTOL = 1e-5
GRAD_COND_TOL = 1e-6
# per test function: [elements, elements within the strict relative bound, max strict relative
# error, max error / term scale] -- printed at the end of the run (pytest_terminal_summary)
GRAD_STATS: dict[str, list] = {}


def assert_grad_close(actual: torch.Tensor, expected: torch.Tensor, term_scale: torch.Tensor) -> None:
    """Gradient parity criterion.  Every element must satisfy

        |actual - expected| <= 1e-5 * |expected|          (relative to the result)
     or |actual - expected| <= 1e-6 * sum_i |t_i|          (for sums whose terms cancel)

    where the t_i are the terms of the sum the gradient consists of and sum |t_i| is computed by
    the fp64 oracle (``absolute=True``).  The second bound is about one fp32 rounding unit of
    the cancellation-free scale: no fp32 evaluation can be asked for more when the signed sum
    is much smaller than its terms."""
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    s = term_scale.detach().double().cpu()
    err = (a - e).abs()
    strict = err <= GRAD_RTOL * e.abs()
    ok = strict | (err <= GRAD_COND_TOL * s)
    name = os.environ.get("PYTEST_CURRENT_TEST", "?").split("::")[-1].split("[")[0].split(" ")[0]
    st = GRAD_STATS.setdefault(name, [0, 0, 0.0, 0.0])
    st[0] += err.numel()
    st[1] += int(strict.sum())
    if err.numel():
        st[2] = max(st[2], float((err / e.abs().clamp_min(1e-300)).max()))
        st[3] = max(st[3], float((err / s.clamp_min(1e-300)).max()))
    assert bool(ok.all()), f"max rel err {float((err / e.abs().clamp_min(1e-300)).max()):.3e}, max err/scale {float((err / s.clamp_min(1e-300)).max()):.3e}"


def device_example(ex: Example, device="cuda:0") -> Example:
    """Move to the device keeping expanded (stride-0) batch dims expanded."""
    def mv(t: torch.Tensor) -> torch.Tensor:
        if any(st == 0 and sz > 1 for st, sz in zip(t.stride(), t.shape)):
            idx = tuple(slice(0, 1) if (st == 0 and sz > 1) else slice(None) for st, sz in zip(t.stride(), t.shape))
            return t[idx].contiguous().to(device).expand(t.shape)
        return t.to(device)

    return Example(mv(ex.x1), mv(ex.x2), mv(ex.rhs), mv(ex.params), mv(ex.start), mv(ex.end), ex.kernel_type, ex.cutoff)


needs_gpu = pytest.mark.gpu
