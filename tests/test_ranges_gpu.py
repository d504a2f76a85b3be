"""Device band construction vs the oracle's restatement of the reference scans: bit-exact."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cases():
    for (m, n, batch) in [(50, 55, ()), (50, 55, (3,)), (50, 55, (2, 3)), (600, 800, ()), (4096, 4096, (2,)), (129, 130, ()), (100, 37, ())]:
        for block in (1, 3, 128):
            for cutoff in (0.1, 1.0, 11.0):
                yield m, n, batch, block, cutoff


@pytest.mark.parametrize("m,n,batch,block,cutoff", list(_cases()))
def test_make_ranges_matches_oracle(m, n, batch, block, cutoff):
    from kernel_matmul_b200 import ranges
    from oracle import oracle as O

    x1 = torch.sort(torch.rand(*batch, m) * 10)[0]
    x2 = torch.sort(torch.rand(*batch, n) * 10)[0] - 1.0
    if m > 20:
        x1[..., 10:] += 20
    for align in (False, True):
        s, e = ranges.make_ranges(cutoff, x1.cuda(), x2.cuda(), block_size=block, align=align)
        rs, re = O.make_ranges(cutoff, x1, x2, block_size=block, align=align)
        assert s.dtype == torch.int32 and s.is_cuda
        assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)
        if align:
            st, et = ranges.transpose_ranges(s, e, m, n, block_size=block)
            rst, ret = O.transpose_ranges(rs, re, m, n, block_size=block)
            assert torch.equal(st.cpu(), rst) and torch.equal(et.cpu(), ret)
    s, e = ranges.make_ranges(cutoff, x1.cuda(), block_size=block)
    rs, re = O.make_ranges(cutoff, x1, block_size=block)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)


def test_unsorted_input_takes_sequential_path():
    from kernel_matmul_b200 import ranges
    from oracle import oracle as O

    x1 = torch.rand(3, 300) * 10
    x2 = torch.rand(3, 280) * 10  # not sorted
    x2[1] = torch.sort(x2[1])[0]  # one sorted batch row among unsorted ones
    for block in (3, 128):
        for align in (False, True):
            s, e = ranges.make_ranges(1.0, x1.cuda(), x2.cuda(), block_size=block, align=align)
            rs, re = O.make_ranges(1.0, x1, x2, block_size=block, align=align)
            assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)
        s, e = ranges.make_ranges(1.0, x1.cuda(), block_size=block)
        rs, re = O.make_ranges(1.0, x1, block_size=block)
        assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)


def test_no_cutoff_and_errors():
    from kernel_matmul_b200 import ranges

    x1 = torch.rand(2, 50).cuda()
    x2 = torch.rand(2, 55).cuda()
    s, e = ranges.make_ranges(None, x1, x2, block_size=3)
    assert torch.all(s == 0) and torch.all(e == 55) and s.shape == (2, 17)
    a = torch.tensor([[0.0, 0.0, 2.0]]).cuda()
    b = torch.tensor([[0.0, 2.0, 2.0]]).cuda()
    s, e = ranges.make_ranges(1.0, a, b, block_size=2, align=False)
    with pytest.raises(ValueError, match="Ranges must be block-aligned"):
        ranges.transpose_ranges(s, e, 3, 3, block_size=2)


def test_symmetric_ranges_with_per_batch_cutoffs():
    """One call with B cutoffs == B calls with one cutoff each (shared and per-batch x, sorted
    and unsorted rows), bit for bit."""
    from kernel_matmul_b200 import ranges

    cutoffs = torch.tensor([0.3, 1.0, 2.5, 7.0, 20.0])
    x = torch.sort(torch.rand(1000) * 10)[0]
    s, e = ranges.make_ranges_symmetric_cutoffs(cutoffs.cuda(), x.cuda())
    for b, c in enumerate(cutoffs.tolist()):
        rs, re_ = ranges.make_ranges(c, x.cuda())
        assert torch.equal(s[b], rs) and torch.equal(e[b], re_)
    xb = torch.sort(torch.rand(5, 700) * 10)[0]
    xb[3] = torch.rand(700) * 10  # an unsorted row takes the sequential scan
    s, e = ranges.make_ranges_symmetric_cutoffs(cutoffs.cuda(), xb.cuda())
    for b, c in enumerate(cutoffs.tolist()):
        rs, re_ = ranges.make_ranges(c, xb[b].cuda())
        assert torch.equal(s[b], rs) and torch.equal(e[b], re_)


def test_dynamic_cutoff_from_a_device_resident_lengthscale():
    # The GPyTorch-facing kernels derive the cutoff from the largest lengthscale
    # (kernel_matmul/gpytorch/base.py:59-64).  Computed on the device (double product, rounded to
    # fp32) and fed to the batched band construction it must give the band of the host-side value.
    import math

    from kernel_matmul_b200 import ranges

    torch.manual_seed(3)
    x = torch.sort(torch.rand(5000) * 40)[0].cuda()
    for eps in (1e-3, 1e-5, 1e-7):
        z = math.sqrt(2.0) * torch.special.erfinv(torch.tensor(1.0 - eps)).item()
        lengthscales = (0.3 + torch.rand(4) * 2).cuda()
        on_device = (lengthscales.max().double() * z).float()
        start_d, end_d = ranges.make_ranges_symmetric_cutoffs(on_device.reshape(1), x)
        start_h, end_h = ranges.make_ranges(z * lengthscales.max().item(), x, align=True)
        assert torch.equal(start_d[0], start_h) and torch.equal(end_d[0], end_h)
