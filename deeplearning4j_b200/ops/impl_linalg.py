"""Linear-algebra ops (``headers/blas.h`` svd/sqrtm + linalg entries of ``headers/parity_ops.h``):
the reference wraps cuSOLVER (``helpers/cuda/svd.cu``, ``lup.cu``); here ``torch.linalg``."""
from __future__ import annotations

import torch

from .registry import op


@op("svd", n_out=-1)
def svd(x, fullUV=False, computeUv=True, switchNum=16, **kw):
    if not computeUv:
        return (torch.linalg.svdvals(x),)
    u, s, vh = torch.linalg.svd(x, full_matrices=bool(fullUV))
    return s, u, vh.transpose(-1, -2)


op("sqrtm")(lambda x, **kw: _sqrtm(x))


def _sqrtm(a):
    w, v = torch.linalg.eig(a.to(torch.float64))
    r = (v * torch.sqrt(w).unsqueeze(-2)) @ torch.linalg.inv(v)
    return r.real.to(a.dtype)


op("matrix_determinant")(lambda x, **kw: torch.linalg.det(x))
op("log_matrix_determinant", n_out=2)(lambda x, **kw: tuple(torch.linalg.slogdet(x)))
op("logdet")(lambda x, **kw: torch.linalg.slogdet(x)[1])
op("matrix_inverse")(lambda x, **kw: torch.linalg.inv(x))
op("cholesky")(lambda x, **kw: torch.linalg.cholesky(x))
op("qr", n_out=2)(lambda x, fullMatricies=False, **kw: tuple(torch.linalg.qr(x, mode="complete" if fullMatricies else "reduced")))


@op("lu", n_out=2)
def lu(x, **kw):
    LU, piv = torch.linalg.lu_factor(x)
    # native op returns the permutation vector (not LAPACK pivots)
    n = x.shape[-1]
    perm = torch.arange(n, device=x.device).expand(x.shape[:-2] + (n,)).clone()
    pv = (piv - 1).long()
    for i in range(n):
        j = pv[..., i:i + 1]
        a = perm[..., i:i + 1].clone()
        b = perm.gather(-1, j)
        perm.scatter_(-1, j, a)
        perm[..., i:i + 1] = b
    return LU, perm.to(torch.int32)


@op("triangular_solve")
def triangular_solve(a, b, lower=True, adjoint=False, **kw):
    A = a.transpose(-1, -2) if adjoint else a
    return torch.linalg.solve_triangular(A, b, upper=not (bool(lower) ^ bool(adjoint)))


op("solve")(lambda a, b, adjoint=False, **kw: torch.linalg.solve(a.transpose(-1, -2) if adjoint else a, b))


@op("lstsq", "solve_ls")
def lstsq(a, b, l2Regularizer=0.0, fast=True, **kw):
    if l2Regularizer:
        at = a.transpose(-1, -2)
        eye = torch.eye(a.shape[-1], dtype=a.dtype, device=a.device)
        return torch.linalg.solve(at @ a + l2Regularizer * eye, at @ b)
    return torch.linalg.lstsq(a, b).solution


@op("eig", n_out=2)
def eig(x, **kw):
    w, v = torch.linalg.eig(x)
    return torch.view_as_real(w), torch.view_as_real(v)


op("self_adjoint_eig", n_out=2)(lambda x, **kw: tuple(torch.linalg.eigh(x)))
op("matrix_power")(lambda x, n=1, **kw: torch.linalg.matrix_power(x, int(n)))
op("pinv")(lambda x, **kw: torch.linalg.pinv(x))
op("knn_mindistance")(lambda point, lowest, highest, **kw: torch.sqrt(
    (torch.clamp(lowest - point, min=0) ** 2 + torch.clamp(point - highest, min=0) ** 2).sum()))
