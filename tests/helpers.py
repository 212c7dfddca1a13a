import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def rel_l2(a, b) -> float:
    """||a-b|| / ||b|| in float64."""
    a = torch.as_tensor(a).detach().cpu().double()
    b = torch.as_tensor(b).detach().cpu().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name))
    data = {k: torch.from_numpy(z[k]) for k in z.files if not k.startswith('p_')}
    params = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith('p_')}
    return data, params
