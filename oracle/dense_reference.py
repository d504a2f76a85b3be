"""The reference's dense PyTorch formulation: materialise K, mask by ranges, matmul.

TEST INFRASTRUCTURE ONLY (see ``km_oracle.c``).  This is the formulation the reference's own
tests compare its CUDA kernels against (tests/conftest.py:163-254): build the full kernel
matrix with torch ops, copy the column range ``[start[r], end[r])`` of every 128-row block
into a zero matrix (tests/conftest.py:243-249) and multiply; hyper-parameter gradients come
from autograd through that graph (tests/native/test_matmul_bwd.py:26-27,
tests/native/test_bilinear_derivative.py:35-40).

The reference builds K with GPyTorch kernel modules (tests/conftest.py:179-226); GPyTorch is
not available here, so K is written in closed form from the same parametrisation:

* rbf               ``s * exp(-tau^2 / (2 l^2))``                   (ScaleKernel(RBFKernel))
* spectral          ``s * exp(-tau^2 / (2 l^2)) * cos(2 pi f tau)``  (SpectralMixtureKernel with
                    one mixture, scale 1/(2 pi l), mean f, weight s; conftest.py:187-200)
* locally_periodic  ``s * exp(-tau^2 / (2 l_r^2)) * exp(-2 sin^2(pi tau / p) / l_p)``
                    (ScaleKernel(RBFKernel * PeriodicKernel); conftest.py:201-226)

which are the values native/common/kernel_function.cuh:25-58 computes after
``transform_params`` (kernel_function.cuh:198-219).

It serves two purposes: in fp64 it is a second, independent oracle (autograd instead of
hand-written partials) that the C oracle is cross-checked against, and in fp32 with all host
threads it is the timed CPU baseline.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

BLOCK_SIZE = 128


def kernel_matrix(kernel_type: str, x1: Tensor, x2: Tensor, params: Tensor) -> Tensor:
    """K[..., i, j] for x1 (..., m), x2 (..., n), params (..., P); dtype follows the inputs."""
    tau = x1[..., :, None] - x2[..., None, :]
    p = params[..., None, None, :]
    if kernel_type == "rbf":
        lengthscale, outputscale = p[..., 0], p[..., 1]
        return outputscale * torch.exp(-0.5 * (tau / lengthscale) ** 2)
    if kernel_type == "spectral":
        lengthscale, frequency, outputscale = p[..., 0], p[..., 1], p[..., 2]
        return (
            outputscale
            * torch.exp(-0.5 * (tau / lengthscale) ** 2)
            * torch.cos(2 * math.pi * frequency * tau)
        )
    if kernel_type == "locally_periodic":
        l_rbf, l_per, period, outputscale = p[..., 0], p[..., 1], p[..., 2], p[..., 3]
        rbf = torch.exp(-0.5 * (tau / l_rbf) ** 2)
        periodic = torch.exp(-2.0 * torch.sin(math.pi * tau / period) ** 2 / l_per)
        return outputscale * rbf * periodic
    raise ValueError(f"Unknown kernel type: {kernel_type}")


def band_mask(start: Tensor, end: Tensor, m: int, n: int, block: int = BLOCK_SIZE) -> Tensor:
    """Boolean (..., m, n) mask: row block r keeps columns [start[..., r], end[..., r])."""
    cols = torch.arange(n, device=start.device)
    rows = torch.arange(m, device=start.device) // block
    s = start.to(torch.int64)[..., rows]  # (..., m)
    e = end.to(torch.int64)[..., rows]
    return (cols >= s[..., None]) & (cols < e[..., None])


def masked_kernel(kernel_type, x1, x2, params, start, end, *, block=BLOCK_SIZE, dtype=torch.float64):
    K = kernel_matrix(kernel_type, x1.to(dtype), x2.to(dtype), params.to(dtype))
    mask = band_mask(start, end, x1.shape[-1], x2.shape[-1], block)
    return torch.where(mask, K, torch.zeros((), dtype=dtype))


def matmul(kernel_type, x1, x2, rhs, params, start, end, *, block=BLOCK_SIZE, dtype=torch.float64):
    return masked_kernel(kernel_type, x1, x2, params, start, end, block=block, dtype=dtype) @ rhs.to(dtype)


def matmul_bwd(kernel_type, x1, x2, rhs, params, start, end, out_grad, *, block=BLOCK_SIZE, dtype=torch.float64):
    p = params.detach().to(dtype).clone().requires_grad_(True)
    out = masked_kernel(kernel_type, x1, x2, p, start, end, block=block, dtype=dtype) @ rhs.to(dtype)
    out.backward(gradient=out_grad.to(dtype).expand_as(out))
    return p.grad


def bilinear_derivative(kernel_type, x1, x2, left, right, params, start, end, *, block=BLOCK_SIZE, dtype=torch.float64):
    p = params.detach().to(dtype).clone().requires_grad_(True)
    K = masked_kernel(kernel_type, x1, x2, p, start, end, block=block, dtype=dtype)
    total = (left.to(dtype) * (K @ right.to(dtype))).sum()
    total.backward()
    return p.grad


def dense_bwd(kernel_type, x1, x2, params, start, end, out_grad, *, block=BLOCK_SIZE, dtype=torch.float64):
    p = params.detach().to(dtype).clone().requires_grad_(True)
    K = masked_kernel(kernel_type, x1, x2, p, start, end, block=block, dtype=dtype)
    K.backward(gradient=out_grad.to(dtype).expand_as(K))
    return p.grad


def matmul_slabs(kernel_type, x1, x2, rhs, params, start, end, *, block=BLOCK_SIZE,
                 dtype=torch.float32, blocks_per_slab: int = 16, row_blocks=None) -> Tensor:
    """Same product for sizes where the full K does not fit: groups of row blocks are
    materialised against only the columns any block of the group can touch.  Masked entries are
    exact zeros, so the result equals the full dense formulation.  Unbatched inputs
    (x1 (m,), x2 (n,), rhs (n,k), params (P,), start/end (R,)).  ``row_blocks`` restricts the
    computation to a subset (the rest of the output stays zero)."""
    m, n = x1.shape[-1], x2.shape[-1]
    R = start.shape[-1]
    out = torch.zeros(m, rhs.shape[-1], dtype=dtype)
    todo = list(range(R)) if row_blocks is None else sorted(int(r) for r in row_blocks)
    rhs_t = rhs.to(dtype)
    i = 0
    while i < len(todo):
        group = [todo[i]]
        while i + len(group) < len(todo) and len(group) < blocks_per_slab and todo[i + len(group)] == group[-1] + 1:
            group.append(todo[i + len(group)])
        i += len(group)
        r0, r1 = group[0], group[-1] + 1
        c0 = int(start[r0:r1].min())
        c1 = min(int(end[r0:r1].max()), n)
        if c1 <= c0:
            continue
        rows = slice(r0 * block, min(r1 * block, m))
        K = kernel_matrix(kernel_type, x1[rows].to(dtype), x2[c0:c1].to(dtype), params.to(dtype))
        mask = band_mask(start[r0:r1] - c0, end[r0:r1] - c0, K.shape[0], c1 - c0, block)
        K = torch.where(mask, K, torch.zeros((), dtype=dtype))
        out[rows] = K @ rhs_t[c0:c1]
    return out
