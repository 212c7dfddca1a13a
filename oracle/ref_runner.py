"""The CPU baseline of the benchmark: the reference's own GalerkinTransformer2D when oracle/_ref holds it (see
oracle/build_ref.py), else the restatement in oracle/gt_oracle.py.  TEST / MEASUREMENT INFRASTRUCTURE ONLY.

Nothing here imports the product package, so a process that only runs this baseline never maps the CUDA library.
"""
from __future__ import annotations

import os
import sys
from typing import Callable, Dict, Tuple

import numpy as np
import torch

from . import gt_oracle as O

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), '_ref')
_DROPS = ('drop_module', 'drop_downscaler', 'drop_upscaler', 'drop_encoder_attn', 'drop_encoder_attn_fc', 'drop_encoder_ffn',
          'drop_decoder_layer')


class _UnitNormalizer:
    """Target normaliser with mean 0 and standard deviation 1, as the reference's GaussNormalizer() default
    (dataset/darcy_dataset.py:23-31): inverse_transform(X) = X * (std + 1e-5) + mean."""

    def inverse_transform(self, X):
        return X * (1.0 + 1.0e-5) + 0.0


def spgt_to_gt_state(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """SpGT parameter layouts -> GT layouts: Q/K/V matrices transposed (x W vs F.linear), Fourier weights
    [m, m, in, out, 2] -> [in, out, m, m, 2]  (network/sp_layer.py:119-121 vs network/layer.py:214-216)."""
    out = {}
    for k, v in state.items():
        v = v.detach().clone()
        if k.split('.')[-1] in ('weight_Q', 'weight_K', 'weight_V'):
            v = v.t().contiguous()
        if 'fourier_weight' in k:
            v = v.permute(2, 3, 0, 1, 4).contiguous()
        out[k] = v
    return out


def synthetic_batch(indices, fine_resolution: int, sub_node: int, sub_attn: int, seed: int) -> Dict[str, torch.Tensor]:
    """The benchmark's synthetic samples for the given global indices (a sample depends on (seed, index) only): thresholded
    Gaussian random fields (dataset/darcy_generate/Gaussian_Random_Field.m:10-19, Darcy_Gen.m:35-37), normalised with the
    analytic mean 7.5 and standard deviation 4.5 of the two-valued field; position / grid as dataset/darcy_dataset.py:117-127."""
    fields = []
    for i in indices:
        U = O.gaussian_random_field(fine_resolution, np.random.default_rng([seed, int(i)]))
        fields.append(np.where(U >= 0, 12.0, 3.0)[::sub_node, ::sub_node])
    a = np.stack(fields).astype(np.float32)[..., None]
    n = a.shape[0]
    node = (a - 7.5) / (4.5 + 1.0e-5)
    pos = O.meshgrid(fine_resolution, sub_attn).astype(np.float32)
    grid = O.meshgrid(fine_resolution, sub_node).astype(np.float32)
    return dict(node=torch.from_numpy(node.astype(np.float32)),
                position=torch.from_numpy(np.broadcast_to(pos, (n, *pos.shape)).copy()),
                grid=torch.from_numpy(np.broadcast_to(grid, (n, *grid.shape)).copy()))


def make_forward(ocfg: dict, spgt_state: Dict[str, torch.Tensor]) -> Tuple[Callable, str]:
    """(forward(node, position, grid) -> prediction, kind).  kind is "reference" when the forward is the reference's own
    GalerkinTransformer2D (network/model.py:126-172) loaded with the given weights, "port" when it is the restatement."""
    if os.path.isfile(os.path.join(_REF, 'SpGT', 'network', 'model.py')):
        if _REF not in sys.path:
            sys.path.insert(0, _REF)
        from SpGT.network.model import GalerkinTransformer2D       # the reference's file, unmodified
        cfg = dict(ocfg)
        for k in _DROPS:
            cfg[k] = 0.0
        cfg['target_normalizer'] = _UnitNormalizer()
        model = GalerkinTransformer2D(cfg).eval()
        model.load_state_dict(spgt_to_gt_state(spgt_state), strict=True)

        def fwd(node, position, grid):
            with torch.no_grad():
                return model(node, position, grid)
        return fwd, 'reference'

    def fwd(node, position, grid):
        with torch.no_grad():
            return O.model_forward(node, position, grid, spgt_state, ocfg)
    return fwd, 'port'
