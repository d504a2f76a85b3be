"""CPU tests of the checker itself: the oracle against fixtures produced by the reference's
own code, and the two independent restatements against each other."""
import os

import numpy as np
import pytest
import torch

from conftest import KERNEL_TYPES, SHAPES, make_example

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ranges_golden.npz")


@pytest.fixture(scope="module")
def O():
    from oracle import oracle

    return oracle


@pytest.fixture(scope="module")
def D():
    from oracle import dense_reference

    return dense_reference


def test_band_oracle_matches_reference_golden(O):
    """oracle/km_oracle.c vs outputs of the reference's native/ranges/ranges.cpp (bit-exact)."""
    g = np.load(GOLDEN)
    meta = g["meta"]
    assert len(meta) > 400
    pos = {f: 0 for f in ("start", "end", "start_t", "end_t", "sym_start", "sym_end")}

    def take(field, shape):
        n = int(np.prod(shape))
        out = g[field][pos[field] : pos[field] + n].reshape(shape)
        pos[field] += n
        return out

    for case, (cutoff, block, align, inp) in enumerate(meta):
        block, align, inp = int(block), bool(align), int(inp)
        x1 = torch.from_numpy(g[f"in{inp}_x1"])
        x2 = torch.from_numpy(g[f"in{inp}_x2"])
        B, m, n = x1.shape[0], x1.shape[1], x2.shape[1]
        R, C = -(-m // block), -(-n // block)
        s, e = O.make_ranges(float(cutoff), x1, x2, block_size=block, align=align)
        assert np.array_equal(s.numpy(), take("start", (B, R))), case
        assert np.array_equal(e.numpy(), take("end", (B, R))), case
        if align:
            st, et = O.transpose_ranges(s, e, m, n, block_size=block)
            assert np.array_equal(st.numpy(), take("start_t", (B, C))), case
            assert np.array_equal(et.numpy(), take("end_t", (B, C))), case
        ss, se = O.make_ranges(float(cutoff), x1, block_size=block)
        assert np.array_equal(ss.numpy(), take("sym_start", (B, R))), case
        assert np.array_equal(se.numpy(), take("sym_end", (B, R))), case
    for f, p in pos.items():
        assert p == len(g[f]), f


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "km_ref_ranges", "km_ref_ranges.so")),
                    reason="reference band module not built (oracle/build_ref.py)")
def test_band_oracle_matches_live_reference(O):
    """Same comparison against the compiled reference module on fresh random inputs."""
    from golden.make_ranges_golden import load_ref

    ref = load_ref()
    for trial in range(20):
        B, m, n = 1 + trial % 3, 40 + 37 * trial, 50 + 29 * trial
        x1 = torch.sort(torch.rand(B, m) * 10)[0]
        x2 = torch.sort(torch.rand(B, n) * 10)[0]
        if trial % 4 == 3:  # unsorted inputs follow the same sequential scan
            x2 = torch.rand(B, n) * 10
        for block in (1, 3, 128):
            for align in (False, True):
                s, e = O.make_ranges(0.7, x1, x2, block_size=block, align=align)
                rs, re = ref.make_ranges(x1, x2, 0.7, block, align)
                assert torch.equal(s, rs) and torch.equal(e, re)
            s, e = O.make_ranges(0.7, x1, block_size=block)
            rs, re = ref.make_ranges_symmetric(x1, 0.7, block)
            assert torch.equal(s, rs) and torch.equal(e, re)


CASES = [pytest.param(s, kt, id=f"shape{i}-{kt}") for i, s in enumerate(SHAPES) for kt in KERNEL_TYPES]


@pytest.mark.parametrize("shape,kt", CASES)
def test_c_oracle_matches_dense_formulation(O, D, shape, kt):
    """Hand-written partials in C (km_oracle.c) vs autograd through the masked dense torch
    formulation (dense_reference.py), both fp64."""
    ex = make_example(shape, kt)
    a = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    b = D.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    assert float((a - b).abs().max()) <= 1e-12 * max(1.0, float(b.abs().max()))
    og = torch.randn(*ex.params.shape[:-1], ex.x1.shape[-1], ex.rhs.shape[-1])
    ga = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    gb = D.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    scale = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og, absolute=True)
    assert bool(((ga - gb).abs() <= 1e-12 * scale + 1e-300).all())
    left = torch.randn(*ex.x1.shape, 5)
    right = torch.randn(*ex.x2.shape, 5)
    ga = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    gb = D.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    scale = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end, absolute=True)
    assert bool(((ga - gb).abs() <= 1e-12 * scale + 1e-300).all())
    Kd = O.dense(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end)
    Kt = D.masked_kernel(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end)
    assert float((Kd - Kt).abs().max()) <= 1e-13
    dg = torch.randn_like(Kt, dtype=torch.float32)
    ga = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, dg)
    gb = D.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, dg)
    scale = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, dg, absolute=True)
    assert bool(((ga - gb).abs() <= 1e-12 * scale + 1e-300).all())


def test_oracle_row_block_subset(O):
    ex = make_example(SHAPES[1], "spectral")
    full = O.matmul("spectral", ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    sub = O.matmul("spectral", ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, row_blocks=[4, 1])
    assert torch.equal(sub[1], full[128:256])
    assert torch.equal(sub[0, : 600 - 512], full[512:600])


def test_slab_formulation_equals_full(D):
    ex = make_example(dict(m=1000, n=1000, batch=(), unsqueeze=None, k=4, cutoff=1.0), "spectral", square=True)
    full = D.matmul("spectral", ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, dtype=torch.float64)
    slab = D.matmul_slabs("spectral", ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, dtype=torch.float64, blocks_per_slab=3)
    assert float((full - slab).abs().max()) <= 1e-13


def test_index_oracle_matches_dense(O):
    ex = make_example(SHAPES[2], "locally_periodic", square=True)
    K = O.dense("locally_periodic", ex.x1, ex.x2, ex.params, ex.start, ex.end)
    b = torch.randint(0, 3, (5, 40), dtype=torch.int32)
    r = torch.randint(0, 500, (5, 40), dtype=torch.int32)
    c = torch.randint(0, 500, (5, 40), dtype=torch.int32)
    v = O.index("locally_periodic", ex.x1, ex.x2, ex.params, ex.start, ex.end, (b,), r, c)
    assert torch.equal(v, K[b.long(), r.long(), c.long()])


CUDA_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cuda_golden.npz")


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_oracle_matches_reference_cuda_golden(O, kt):
    """The fp64 oracle vs the fp32 outputs of the reference's own CUDA kernels (compiled
    unmodified, run on a B200; tests/golden/make_cuda_golden.py).  The reference computes in
    fp32, so agreement is to fp32 accuracy: 1e-5 relative for values, and for gradients 1e-4
    relative or 1e-5 of the sum of term magnitudes (its own tests accept 2e-3)."""
    g = np.load(CUDA_GOLDEN)
    t = lambda name: torch.from_numpy(g[f"{kt}_{name}"])  # noqa: E731
    x1, x2, params, start, end = t("x1"), t("x2"), t("params"), t("start"), t("end")

    def close(actual, ref):
        return float((actual - ref.double()).abs().max() / ref.double().abs().max())

    def grad_close(actual, ref, scale):
        err = (actual - ref.double()).abs()
        return bool(((err <= 1e-4 * actual.abs()) | (err <= 1e-5 * scale)).all())

    assert close(O.matmul(kt, x1, x2, t("rhs"), params, start, end), t("ref_matmul")) <= 1e-5
    a = O.matmul_bwd(kt, x1, x2, t("rhs"), params, start, end, t("og"))
    s = O.matmul_bwd(kt, x1, x2, t("rhs"), params, start, end, t("og"), absolute=True)
    assert grad_close(a, t("ref_matmul_bwd"), s)
    a = O.bilinear_derivative(kt, x1, x2, t("left"), t("right"), params, start, end)
    s = O.bilinear_derivative(kt, x1, x2, t("left"), t("right"), params, start, end, absolute=True)
    assert grad_close(a, t("ref_bilinear"), s)
    x1d, x2d = x1[:, :160].contiguous(), x2[:, :150].contiguous()
    dstart, dend = t("dstart"), t("dend")
    K = O.dense(kt, x1d, x2d, params, dstart, dend)
    Kref = t("ref_dense")
    assert close(K, Kref) <= 1e-5
    assert torch.equal(K == 0, Kref == 0)
    a = O.dense_bwd(kt, x1d, x2d, params, dstart, dend, t("dg"))
    s = O.dense_bwd(kt, x1d, x2d, params, dstart, dend, t("dg"), absolute=True)
    assert grad_close(a, t("ref_dense_bwd"), s)
    sstart, send = t("sstart"), t("send")
    v = O.index(kt, x1, x1, params, sstart, send, (t("bidx"),), t("row"), t("col"))
    vref = t("ref_index")
    assert close(v, vref) <= 1e-5
    assert torch.equal(v == 0, vref == 0)  # band membership of every lookup
    a = O.index_bwd(kt, x1, x1, params, sstart, send, (t("bidx"),), t("row"), t("col"), t("ig"))
    s = O.index_bwd(kt, x1, x1, params, sstart, send, (t("bidx"),), t("row"), t("col"), t("ig"), absolute=True)
    assert grad_close(a, t("ref_index_bwd"), s)
    # the band the GPU box computed with the reference's ranges.cpp equals the oracle's
    rs, re = O.make_ranges(2.0, x1, x2)
    assert torch.equal(rs, start) and torch.equal(re, end)
    rs, re = O.make_ranges(2.0, x1)
    assert torch.equal(rs, sstart) and torch.equal(re, send)
