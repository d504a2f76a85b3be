"""The allocation-free gradient entry point against the workspace-taking one.

``km_bilinear_derivative_static_f32`` is for hosts that cannot give the library a workspace
(all device memory already belongs to their own pool, or allocation calls are banned where the
gradient is needed); it keeps its partial sums in an array built into the library.  Both entry
points are called here directly through the C ABI on the same device buffers, twice in a row
(the built-in array is reused and keeps the previous call's contents), and must agree.  The
file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _view(t, nb):
    from kernel_matmul_b200._lib import KmView

    v = KmView()
    v.data = t.data_ptr()
    st = t.stride()
    nbatch = t.dim() - nb
    for d in range(nbatch):
        v.batch_stride[d] = st[d]
    for d in range(nb):
        v.stride[d] = st[nbatch + d]
    return v


@pytest.mark.parametrize("kt,P", [("rbf", 2), ("spectral", 3), ("locally_periodic", 4)])
def test_static_scratch_entry_point_matches_workspace_entry_point(kt, P):
    from kernel_matmul_b200._lib import KERNEL_TYPES, KmBatch, lib
    from oracle import oracle as O

    dev = torch.device("cuda:0")
    B, m, n, k = 3, 700, 650, 7
    x1 = torch.sort(torch.rand(B, m) * 12)[0]
    x2 = torch.sort(torch.rand(B, n) * 12)[0]
    params = 1 + torch.rand(B, P)
    start, end = O.make_ranges(1.5, x1, x2)
    batch = KmBatch()
    batch.ndim = 1
    batch.size[0] = B
    kid = KERNEL_TYPES[kt]
    d = [t.to(dev) for t in (x1, x2, params, start, end)]
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    for call in range(2):  # the second call meets the scratch contents the first one left
        left = torch.randn(B, m, k)
        right = torch.randn(B, n, k)
        dl, dr = left.to(dev), right.to(dev)
        views = (_view(d[0], 1), _view(d[1], 1), _view(dl, 2), _view(dr, 2), _view(d[2], 1), _view(d[3], 1), _view(d[4], 1))
        g_ws = torch.full((B, P), float("nan"), device=dev)
        g_static = torch.full((B, P), float("nan"), device=dev)
        ws_bytes = lib.km_grad_workspace_bytes(kid, batch, m)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        rc = lib.km_bilinear_derivative_f32(kid, batch, m, n, k, *views, _view(g_ws, 1),
                                            ctypes.c_void_p(ws.data_ptr()), ws_bytes, stream)
        assert rc == 0, lib.km_last_error()
        rc = lib.km_bilinear_derivative_static_f32(kid, batch, m, n, k, *views, _view(g_static, 1), stream)
        assert rc == 0, lib.km_last_error()
        torch.cuda.synchronize()
        # same kernels, same summation order: identical bits
        assert torch.equal(g_ws, g_static), (call, g_ws, g_static)
        # and both within the gradient tolerance of the oracle
        from conftest import assert_grad_close

        ref = O.bilinear_derivative(kt, x1, x2, left, right, params, start, end)
        scale = O.bilinear_derivative(kt, x1, x2, left, right, params, start, end, absolute=True)
        assert_grad_close(g_static, ref, scale)


def test_static_scratch_entry_point_refuses_oversized_problems():
    from kernel_matmul_b200._lib import KmBatch, KmView, lib

    batch = KmBatch()
    batch.ndim = 1
    batch.size[0] = 64
    v = KmView()
    # 64 batches x 2^22 rows = 2^21 row-block records > 262144: refused before any launch
    rc = lib.km_bilinear_derivative_static_f32(0, batch, 1 << 22, 1 << 22, 8, v, v, v, v, v, v, v, v, None)
    assert rc == 2
    assert b"exceeds the built-in scratch" in lib.km_last_error()
