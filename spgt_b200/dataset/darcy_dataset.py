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


def central_diff(X: np.ndarray, S: int):
    """Central differences of [N, S, S] fields with zero padding, scaled by S (dataset/darcy_dataset.py:146-154)."""
    X = np.pad(X, pad_width=[(0, 0), (1, 1), (1, 1)], mode='constant', constant_values=0)
    grad_x = (X[:, 2:, 1:-1] - X[:, :-2, 1:-1]) / 2
    grad_y = (X[:, 1:-1, 2:] - X[:, 1:-1, :-2]) / 2
    return grad_x * S, grad_y * S


class DarcyDataset(torch.utils.data.Dataset):
    """The reference's Darcy dataset (dataset/darcy_dataset.py:48-175) for the inference path: coefficient `a` and
    solution `u` of shape [N, R, R] from a .mat file (or a dict holding those arrays), every sub-th node kept, the coefficient normalised per node.

    Items are dicts of float32 tensors: grid [r,r,2], position [r_attn,r_attn,2], coeff [r,r,1] (raw coefficient),
    node [r,r,1] (normalised), target [r,r,1], target_grad [r,r,2].  Training sets take the first num_data samples
    and fit the normalisers; validation sets take the last num_data samples and need the training node_normalizer."""

    def __init__(self, datapath, subsample_node, subsample_attn=None, num_data=None, fine_resolution=None,
                 is_training=True, is_return_boundary=True, is_normalization=True, node_normalizer: GaussNormalizer = None,
                 noise=0.0, random_seed=1127802, keys=('a', 'u')) -> None:
        super().__init__()
        from .data_accessor import read_matfile
        self.datapath, self.is_training = datapath, is_training
        self.subsample_node = subsample_node
        self.subsample_attn = subsample_attn if subsample_attn is not None else 2 * subsample_node
        self.is_return_boundary, self.is_normalization = is_return_boundary, is_normalization
        self.node_normalizer, self.target_normalizer = node_normalizer, None
        if isinstance(datapath, dict):            # in-memory samples, e.g. from dataset.darcy_generate.generate()
            a, u = (np.asarray(datapath[k], dtype=np.float32) for k in keys)
        else:
            a, u = read_matfile(datapath, list(keys), [np.float32, np.float32])
        N, R, _ = a.shape
        self.num_data = num_data if num_data is not None else N
        self.fine_resolution = fine_resolution if fine_resolution is not None else R
        if is_training:
            a, u = a[:self.num_data], u[:self.num_data]
        else:
            a, u = a[-self.num_data:], u[-self.num_data:]
        sub = self.subsample_node
        r = int((R - 1) / sub + 1)
        n = a.shape[0]
        self.grid = meshgrid(R, sub, is_return_boundary)
        self.position = meshgrid(R, self.subsample_attn, True)
        nodes = a[:, ::sub, ::sub].reshape(n, r, r, 1)
        self.targets = u[:, ::sub, ::sub].reshape(n, r, r, 1)
        gx, gy = central_diff(u, R)
        self.targets_grad = np.stack([gx[:, ::sub, ::sub], gy[:, ::sub, ::sub]], axis=-1).reshape(n, r, r, 2)
        self.coeffs = np.copy(nodes)
        if is_normalization:
            if is_training:
                self.node_normalizer = GaussNormalizer(nodes)
                self.target_normalizer = GaussNormalizer(self.targets if is_return_boundary else self.targets[:, 1:-1, 1:-1, :])
            elif self.node_normalizer is None:
                raise ValueError('a validation set needs the node_normalizer fitted on the training set')
            nodes = self.node_normalizer.transform(nodes)
        if noise > 0.0:
            nodes = nodes + noise * np.random.default_rng(random_seed).standard_normal(nodes.shape)
        self.nodes = nodes

    def __len__(self):
        return self.num_data

    def __getitem__(self, index) -> dict:
        return dict(
            grid=torch.from_numpy(self.grid).float(), position=torch.from_numpy(self.position).float(),
            coeff=torch.from_numpy(self.coeffs[index]).float(), node=torch.from_numpy(np.asarray(self.nodes[index])).float(),
            target=torch.from_numpy(self.targets[index]).float(), target_grad=torch.from_numpy(self.targets_grad[index]).float())

    def batches(self, batch_size: int, pin_memory: bool = False):
        """Consecutive batches in the layout HostInference takes (grid and position repeated per sample)."""
        for s in range(0, len(self), batch_size):
            idx = range(s, min(s + batch_size, len(self)))
            items = [self[i] for i in idx]
            batch = {k: torch.stack([it[k] for it in items]) for k in items[0]}
            yield {k: (v.pin_memory() if pin_memory else v) for k, v in batch.items()}
