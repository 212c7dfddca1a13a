"""Synthetic Darcy-flow samples with targets, after the reference's MATLAB generator
(dataset/darcy_generate/{Gaussian_Random_Field,Darcy_Gen,Solve_GWF,gen}.m).

Per sample: a Gaussian random field U (alpha = 2, tau = 3) by an inverse 2-D DCT of scaled white noise, the
coefficient a = 12 where U >= 0 and 3 elsewhere, forcing f = 1, and the solution u of -div(a grad u) = f on the unit
square with u = 0 on the boundary: cubic-spline resampling of a and f from the S x S cell centres to the S x S nodes,
the 5-point finite-volume system on the nodes, and resampling of the solution back to the cell centres.

The random field and the resampling are small host-side array operations (numpy / scipy, float64 as in MATLAB);
the linear systems of a whole batch are solved on the GPU by the library's conjugate-gradient kernels
(`ops.darcy_fv_solve`; the reference calls MATLAB's sparse direct solver).  The output dictionary has the keys of
the reference's .mat files (gen.m:13-27), so `DarcyDataset` reads it like a file.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch


def gaussian_random_field(S: int, rng: np.random.Generator, alpha: float = 2.0, tau: float = 3.0) -> np.ndarray:
    """Gaussian_Random_Field.m:10-19 (covariance (-Laplace + tau^2)^(-alpha), Neumann boundary)."""
    import scipy.fft
    k1, k2 = np.meshgrid(np.arange(S), np.arange(S))
    coef = tau ** (alpha - 1) * (np.pi ** 2 * (k1 ** 2 + k2 ** 2) + tau ** 2) ** (-alpha / 2)
    L = S * coef * rng.standard_normal((S, S))
    L[0, 0] = 0.0
    return scipy.fft.idctn(L, type=2, norm='ortho')


def _resample(Z: np.ndarray, src: np.ndarray, dst: np.ndarray) -> np.ndarray:
    """Tensor-product not-a-knot cubic spline over the last two axes (MATLAB interp2 'spline', Solve_GWF.m:9-10,41)."""
    from scipy.interpolate import CubicSpline
    Z = CubicSpline(src, Z, axis=-2, bc_type='not-a-knot', extrapolate=True)(dst)
    return CubicSpline(src, Z, axis=-1, bc_type='not-a-knot', extrapolate=True)(dst)


def solve_darcy(a: np.ndarray, f: np.ndarray = None, device='cuda', rel_tol: float = 1.0e-10) -> np.ndarray:
    """Solve_GWF.m for a batch: cell-centre coefficients a [B, S, S] (and forcing f, default 1) -> cell-centre
    solutions [B, S, S] (float64)."""
    from .. import ops
    B, S, _ = a.shape
    centres = (2.0 * np.arange(S) + 1.0) / (2.0 * S)
    nodes = np.arange(S) / (S - 1.0)
    f = np.ones_like(a, dtype=np.float64) if f is None else f
    cn = torch.from_numpy(np.ascontiguousarray(_resample(a.astype(np.float64), centres, nodes))).to(device)
    fn = torch.from_numpy(np.ascontiguousarray(_resample(f.astype(np.float64), centres, nodes))).to(device)
    p, _, _ = ops.darcy_fv_solve(cn, fn, rel_tol=rel_tol)
    return _resample(p.cpu().numpy(), nodes, centres)


def generate(num_data: int, S: int, seed: int = 0, device='cuda', batch: int = 16) -> Dict[str, np.ndarray]:
    """num_data samples at resolution S: {'a', 'u', 'a_mean', 'u_mean', 'a_std', 'u_std'} as in gen.m:13-27
    (statistics over the sample axis; MATLAB's std normalises by N - 1)."""
    a = np.empty((num_data, S, S))
    u = np.empty((num_data, S, S))
    for i in range(num_data):
        U = gaussian_random_field(S, np.random.default_rng([seed, i]))
        a[i] = np.where(U >= 0, 12.0, 3.0)                                   # Darcy_Gen.m:35-37
    for i0 in range(0, num_data, batch):
        u[i0:i0 + batch] = solve_darcy(a[i0:i0 + batch], device=device)
    ddof = 1 if num_data > 1 else 0
    return {'a': a, 'u': u, 'a_mean': a.mean(0, keepdims=True), 'u_mean': u.mean(0, keepdims=True),
            'a_std': a.std(0, ddof=ddof, keepdims=True), 'u_std': u.std(0, ddof=ddof, keepdims=True)}


def save_mat(path: str, data: Dict[str, np.ndarray]) -> None:
    """Write the dictionary of `generate` as a MATLAB v5 file with the reference's variable names (the reference saves
    v7.3 / HDF5, gen.m:27; `data_accessor.read_matfile` reads both)."""
    import scipy.io
    scipy.io.savemat(path, data, do_compression=True)
