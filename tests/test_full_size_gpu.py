"""Parity at the sizes of the benchmark configurations.

A dense fp64 K does not fit for n >= 131072, so at full size the CUDA results are compared with
the oracle on sampled row blocks (the oracle evaluates only those blocks), and through
size-independent properties: symmetry of the bilinear form for symmetric bands,
<u, K v> = <v, K u>, and linearity.  Inputs are the seeded workloads of
``kernel_matmul_b200/workloads.py``.
"""
import pytest
import torch

from conftest import assert_grad_close, rel_err

pytestmark = pytest.mark.gpu


def _sample_blocks(R, count, seed=0):
    g = torch.Generator().manual_seed(seed)
    picks = {0, R - 1, R // 2}
    while len(picks) < count:
        picks.add(int(torch.randint(0, R, (1,), generator=g)))
    return sorted(picks)


def test_rbf_small_config_exact_against_full_oracle():
    """The small RBF configuration in full (n = 4096): every output row against the oracle."""
    from kernel_matmul_b200 import ops, workloads
    from oracle import oracle as O

    w = workloads.rbf_small()
    x = w.x.cuda()
    start, end = workloads.band(w, x)
    rs, re = O.make_ranges(w.cutoffs[0], w.x)
    assert torch.equal(start.cpu(), rs) and torch.equal(end.cpu(), re)
    assert O.count_entries(w.n, w.n, rs, re) == int(ops.count_entries(w.n, w.n, start, end)) == 2523136
    out = ops.matmul("rbf", x, x, w.rhs.cuda(), w.params.cuda(), start, end)
    ref = O.matmul("rbf", w.x, w.x, w.rhs, w.params, rs, re)
    assert rel_err(out, ref) <= 1e-5


def test_spectral_mixture_config_every_row_of_the_product():
    """The 16-component spectral mixture (n = 65536, k = 16) in full: every one of the 1 048 576
    output rows x 16 columns against the fp64 oracle (1.76e9 entries, a few tens of seconds of
    CPU), on both kernel families."""
    from kernel_matmul_b200 import ops, workloads
    from oracle import oracle as O

    w = workloads.spectral_mixture()
    B, n, k = w.params.shape[0], w.n, w.rhs.shape[-1]
    x = w.x.cuda()
    start, end = workloads.band(w, x)
    ref = O.matmul("spectral", w.x.expand(B, n), w.x.expand(B, n), w.rhs.expand(B, n, k), w.params, start.cpu(), end.cpu())
    xb = x.expand(B, n)
    for path in ("tc", "fma"):
        out = ops.matmul("spectral", xb, xb, w.rhs.cuda().expand(B, n, k), w.params.cuda(), start, end, path=path)
        ops.check()
        err = (out.cpu().double() - ref).abs()
        assert float(err.max() / ref.abs().max()) <= 1e-5, path
        # per component as well (their scales differ by the lengthscale)
        assert bool((err.amax(dim=(1, 2)) <= 1e-5 * ref.abs().amax(dim=(1, 2))).all()), path


def test_spectral_mixture_config_sampled_blocks_and_properties():
    """The spectral-mixture configuration (16 components, n = 65536, k = 16): forward on sampled row blocks,
    gradient restricted to sampled row blocks, symmetry and linearity on the full product."""
    from kernel_matmul_b200 import ops, workloads
    from oracle import oracle as O

    w = workloads.spectral_mixture()
    B, n, k = w.params.shape[0], w.n, w.rhs.shape[-1]
    x = w.x.cuda()
    start, end = workloads.band(w, x)
    rs = torch.stack([O.make_ranges(c, w.x)[0] for c in w.cutoffs])
    re = torch.stack([O.make_ranges(c, w.x)[1] for c in w.cutoffs])
    assert torch.equal(start.cpu(), rs) and torch.equal(end.cpu(), re)  # band: bit-exact
    xb = x.expand(B, n)
    rhs = w.rhs.cuda().expand(B, n, k)
    params = w.params.cuda()
    out = ops.matmul("spectral", xb, xb, rhs, params, start, end)
    blocks = _sample_blocks(n // 128, 6)
    ref = O.matmul("spectral", w.x.expand(B, n), w.x.expand(B, n), w.rhs.expand(B, n, k), w.params, rs, re, row_blocks=blocks)
    got = torch.stack([out[:, r * 128:(r + 1) * 128] for r in blocks], dim=1)
    assert rel_err(got, ref) <= 1e-5
    # symmetry of the operator (x1 == x2, symmetric band): <u, K v> == <v, K u>
    u = torch.randn(n, k, device="cuda")
    Ku = ops.matmul("spectral", xb, xb, u.expand(B, n, k), params, start, end)
    lhs = (u.double() * out.double()).sum(dim=(1, 2))      # <u, K rhs>
    rhs_ = (w.rhs.cuda().double() * Ku.double()).sum(dim=(1, 2))  # <rhs, K u>
    scale = (u.double().abs() * out.double().abs()).sum(dim=(1, 2))
    assert bool(((lhs - rhs_).abs() <= 1e-5 * scale).all())
    # linearity: K (2 rhs - u) == 2 K rhs - K u
    mix = ops.matmul("spectral", xb, xb, (2 * w.rhs.cuda() - u).expand(B, n, k), params, start, end)
    assert rel_err(mix, 2 * out.double() - Ku.double()) <= 1e-5
    # gradient on sampled row blocks: empty bands everywhere else
    og = w.extra["out_grad"]
    keep = torch.zeros(n // 128, dtype=torch.bool)
    keep[blocks] = True
    s2 = torch.where(keep, rs, re)  # start = end: nothing visited in the other blocks
    g = ops.matmul_bwd("spectral", xb, xb, rhs, params, s2.cuda(), end, og.cuda())
    gref = O.matmul_bwd("spectral", w.x.expand(B, n), w.x.expand(B, n), w.rhs.expand(B, n, k), w.params, s2, re, og)
    gscale = O.matmul_bwd("spectral", w.x.expand(B, n), w.x.expand(B, n), w.rhs.expand(B, n, k), w.params, s2, re, og, absolute=True)
    assert_grad_close(g, gref, gscale)


def test_locally_periodic_bilinear_config_sampled_blocks():
    """The locally periodic configuration (batch 4, n = 262144, k = 32): bilinear_derivative restricted to sampled
    row blocks against the oracle, and the full-size call for shape / finiteness."""
    from kernel_matmul_b200 import ops, workloads
    from oracle import oracle as O

    w = workloads.locally_periodic_bilinear()
    B, n, k = w.params.shape[0], w.n, w.rhs.shape[-1]
    x = w.x.cuda()
    start, end = workloads.band(w, x)
    rs, re = O.make_ranges(w.cutoffs[0], w.x)
    assert torch.equal(start[0].cpu(), rs) and torch.equal(end[0].cpu(), re)
    xb = x.expand(B, n)
    lhs, rhs, params = w.extra["lhs"].cuda(), w.rhs.cuda(), w.params.cuda()
    full = ops.bilinear_derivative("locally_periodic", xb, xb, lhs, rhs, params, start, end)
    assert full.shape == (B, 4) and bool(torch.isfinite(full).all())
    blocks = _sample_blocks(n // 128, 5, seed=3)
    keep = torch.zeros(n // 128, dtype=torch.bool)
    keep[blocks] = True
    s2 = torch.where(keep, rs, re)
    g = ops.bilinear_derivative("locally_periodic", xb, xb, lhs, rhs, params, s2.cuda().expand(B, -1), end)
    args = ("locally_periodic", w.x.expand(B, n), w.x.expand(B, n), w.extra["lhs"], w.rhs, w.params, s2.expand(B, -1), re.expand(B, -1))
    assert_grad_close(g, O.bilinear_derivative(*args), O.bilinear_derivative(*args, absolute=True))


def test_unbanded_rbf_config_sampled_blocks_and_gather():
    """The unbanded RBF configuration (n = 131072 unbanded, k = 128; 2^24 gathers)."""
    from kernel_matmul_b200 import ops, ranges, workloads
    from oracle import oracle as O

    w = workloads.rbf_unbanded()
    n, k = w.n, w.rhs.shape[-1]
    x = w.x.cuda()
    start, end = ranges.make_ranges(None, x)
    params = w.params.cuda()
    out = ops.matmul("rbf", x, x, w.rhs.cuda(), params, start, end)
    blocks = [0, 517, n // 128 - 1]
    ref = O.matmul("rbf", w.x, w.x, w.rhs, w.params, start.cpu(), end.cpu(), row_blocks=blocks)
    got = torch.stack([out[r * 128:(r + 1) * 128] for r in blocks])
    assert rel_err(got, ref) <= 1e-5
    row, col = w.extra["row"], w.extra["col"]
    vals = ops.index("rbf", x, x, params, start, end, (), row.cuda(), col.cuda())
    vref = O.index("rbf", w.x, w.x, w.params, start.cpu(), end.cpu(), (), row, col)
    assert rel_err(vals, vref) <= 1e-5


def test_cg_sum_config_sampled_blocks_and_64bit_offsets():
    """The CG configuration (64 components, n = 2^22, k = 8): the batch-summed product and the
    batched product (whose output has 2.1e9 elements, past int32 offsets) on sampled row blocks."""
    from kernel_matmul_b200 import ops, workloads
    from oracle import oracle as O

    w = workloads.cg_sum_kernel()
    B, n, k = w.params.shape[0], w.n, w.rhs.shape[-1]
    x = w.x.cuda()
    start, end = workloads.band(w, x)
    rs, re = O.make_ranges(w.cutoffs[0], w.x)
    assert torch.equal(start[0].cpu(), rs) and torch.equal(end[0].cpu(), re)
    xb = x.expand(B, n)
    y = w.rhs.cuda()
    params = w.params.cuda()
    blocks = _sample_blocks(n // 128, 4, seed=5)
    ref = O.matmul("spectral", w.x.expand(B, n), w.x.expand(B, n), w.rhs.expand(B, n, k), w.params,
                   rs.expand(B, -1), re.expand(B, -1), row_blocks=blocks)  # (B, blocks, 128, k)
    # batch-summed product on windows around the sampled blocks
    for i, r in enumerate(blocks):
        got = ops.matmul_rows("spectral", xb, xb, y.expand(B, n, k), params, start, end,
                              row_block_begin=r, row_block_count=1, sum_batches=True)
        assert rel_err(got, ref[:, i].sum(0)) <= 1e-5
    # batched product in full: (64, 2^22, 8) output, element offsets beyond 2^31
    out = ops.matmul("spectral", xb, xb, y.expand(B, n, k), params, start, end)
    assert out.numel() >= 2**31
    got = torch.stack([out[:, r * 128:(r + 1) * 128] for r in blocks], dim=1)
    assert rel_err(got[-1], ref[-1]) <= 1e-5  # last batch: highest offsets
    assert rel_err(got, ref) <= 1e-5
