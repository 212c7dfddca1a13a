"""Normaliser, node coordinates and synthetic Darcy coefficient fields.

The reference reads .mat files (dataset/darcy_dataset.py, dataset/data_accessor.py); those files are not
redistributable with this package, so inputs with the same shapes and value distribution are synthesised:
a Gaussian random field with covariance (-Laplacian + tau^2)^(-alpha) sampled through an inverse DCT
(dataset/darcy_generate/Gaussian_Random_Field.m:10-19), thresholded to 12 / 3 (dataset/darcy_generate/Darcy_Gen.m:35-37).
"""
from typing import Union

import numpy as np
import torch


class GaussNormalizer:
    """(x - mean) / (std + eps); same interface as the reference's GaussNormalizer (dataset/darcy_dataset.py:11-45)."""

    def __init__(self, X: Union[np.ndarray, torch.Tensor] = None, eps: float = 1.0e-5):
        self.eps = eps
        self.fit(X)

    def fit(self, X, axis=0):
        if isinstance(X, np.ndarray):
            self.mean, self.std = np.mean(X, axis=axis), np.std(X, axis=axis)
        elif isinstance(X, torch.Tensor):
            self.mean, self.std = torch.mean(X, dim=axis), torch.std(X, dim=axis)
        else:
            self.mean, self.std = np.array([0.0]), np.array([1.0])

    def transform(self, X):
        return (X - self.mean) / (self.std + self.eps)

    def inverse_transform(self, X):
        return X * (self.std + self.eps) + self.mean

    def numpy_to_torch(self, device='cpu'):
        if isinstance(self.mean, np.ndarray):
            self.mean = torch.from_numpy(np.asarray(self.mean)).float().to(device)
        if isinstance(self.std, np.ndarray):
            self.std = torch.from_numpy(np.asarray(self.std)).float().to(device)
        return self


def meshgrid(S: int, sub: int, is_return_boundary: bool = True) -> np.ndarray:
    """[r, r, 2] coordinates (x along the last grid axis) of every sub-th node of an S x S unit grid
    (dataset/darcy_dataset.py:117-127)."""
    x, y = np.meshgrid(np.linspace(0, 1, S), np.linspace(0, 1, S))
    x, y = x[::sub, ::sub], y[::sub, ::sub]
    if not is_return_boundary:
        x, y = x[1:-1, 1:-1], y[1:-1, 1:-1]
    return np.stack([x, y], axis=-1)


def gaussian_random_field(S: int, rng: np.random.Generator, alpha: float = 2.0, tau: float = 3.0) -> np.ndarray:
    import scipy.fft
    k1, k2 = np.meshgrid(np.arange(S), np.arange(S))
    coef = tau ** (alpha - 1) * (np.pi ** 2 * (k1 ** 2 + k2 ** 2) + tau ** 2) ** (-alpha / 2)
    L = S * coef * rng.standard_normal((S, S))
    L[0, 0] = 0.0
    return scipy.fft.idctn(L, type=2, norm='ortho')


def synthetic_darcy_batch(indices, fine_resolution: int, sub_node: int, sub_attn: int, seed: int):
    """Synthetic samples for the given global sample indices: dict of float32 tensors
    node [n,r,r,1] (coefficient normalised with the analytic mean 7.5 / std 4.5 of the two-valued field),
    coeff [n,r,r,1], position [n,ra,ra,2], grid [n,r,r,2].  A sample depends only on (seed, index), so any
    sharding of the index range over ranks sees the same data."""
    fields = []
    for i in indices:
        U = gaussian_random_field(fine_resolution, np.random.default_rng([seed, int(i)]))
        fields.append(np.where(U >= 0, 12.0, 3.0)[::sub_node, ::sub_node])
    a = np.stack(fields).astype(np.float32)[..., None]
    n = a.shape[0]
    node = (a - 7.5) / (4.5 + 1.0e-5)
    pos = meshgrid(fine_resolution, sub_attn).astype(np.float32)
    grid = meshgrid(fine_resolution, sub_node).astype(np.float32)
    return dict(
        node=torch.from_numpy(node.astype(np.float32)), coeff=torch.from_numpy(a),
        position=torch.from_numpy(np.broadcast_to(pos, (n, *pos.shape)).copy()),
        grid=torch.from_numpy(np.broadcast_to(grid, (n, *grid.shape)).copy()))
