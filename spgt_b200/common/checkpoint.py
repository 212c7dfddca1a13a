"""Converting checkpoints between the reference's two model families.

The pure-PyTorch GalerkinTransformer2D ("GT", network/model.py + network/layer.py) and Sp_GalerkinTransformer2D
("SpGT", network/sp_model.py + network/sp_layer.py) share parameter names but not layouts:
  * GT keeps the Q/K/V projections as nn.Linear-style [out, in] matrices; the SpGT ops compute x * W with W [in, out];
  * GT stores Fourier weights as [in, out, m, m, 2] (torch.einsum 'bixy,ioxy'); SpGT as [m, m, in, out, 2].
Everything else is identical, so a checkpoint trained with one family can be served by the other.
"""
from typing import Dict

import torch

_QKV = ('weight_Q', 'weight_K', 'weight_V')


_FOURIER_PERM = (2, 3, 0, 1, 4)      # [in, out, m, m, 2] <-> [m, m, in, out, 2]: the permutation is its own inverse


def _convert(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for key, value in state.items():
        value = value.detach().clone()
        if key.split('.')[-1] in _QKV:
            value = value.t().contiguous()
        if 'fourier_weight' in key:
            value = value.permute(*_FOURIER_PERM).contiguous()
        out[key] = value
    return out


def gt_to_spgt_state(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """GT state_dict -> SpGT state_dict (what Sp_GalerkinTransformer2D.load_state_dict takes)."""
    return _convert(state)


def spgt_to_gt_state(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """SpGT state_dict -> GT state_dict; the same transposes undo themselves."""
    return _convert(state)
