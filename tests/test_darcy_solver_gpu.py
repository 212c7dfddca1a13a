"""The CUDA conjugate-gradient Darcy solver against the oracle's sparse direct solve."""
import numpy as np
import pytest
import torch

from oracle import darcy_solver as D

pytestmark = pytest.mark.gpu


def _fields(B, K, seed):
    cn, fn = [], []
    for i in range(B):
        rng = np.random.default_rng([seed, i])
        a = D.threshold_coefficient(D.gaussian_random_field(K, rng))
        cn.append(D.spline_resample(a, D.centres(K), D.nodes(K)))
        fn.append(1.0 + 0.3 * rng.standard_normal((K, K)))
    return np.stack(cn), np.stack(fn)


@pytest.mark.parametrize('B,K', [(1, 3), (2, 4), (3, 33), (2, 85), (1, 141)])
def test_fv_solve_matches_direct_solver(B, K):
    from spgt_b200 import ops
    cn, fn = _fields(B, K, seed=K)
    dev = torch.device('cuda:0')
    p, iters, rel = ops.darcy_fv_solve(torch.from_numpy(cn).to(dev), torch.from_numpy(fn).to(dev), rel_tol=1e-12)
    assert iters > 0 and max(rel) <= 1e-12
    p2, _, _ = ops.darcy_fv_solve(torch.from_numpy(cn).to(dev), torch.from_numpy(fn).to(dev), rel_tol=1e-12)
    assert torch.equal(p, p2)                                    # fixed-order reductions: bitwise repeatable
    p = p.cpu().numpy()
    for b in range(B):
        ref = D.solve_nodes(cn[b], fn[b])
        assert np.abs(p[b] - ref).max() <= 1e-9 * np.abs(ref).max()
        assert p[b][0].max() == 0 and p[b][:, -1].max() == 0     # Dirichlet frame


def test_iteration_limit_is_reported():
    from spgt_b200 import ops
    cn, fn = _fields(1, 65, seed=1)
    dev = torch.device('cuda:0')
    with pytest.raises(RuntimeError, match='iteration limit'):
        ops.darcy_fv_solve(torch.from_numpy(cn).to(dev), torch.from_numpy(fn).to(dev), rel_tol=1e-12, max_iter=5, check_every=5)


def test_generate_matches_oracle_samples():
    from spgt_b200.dataset import darcy_generate as G
    data = G.generate(3, 43, seed=7, batch=2)
    assert data['a'].shape == (3, 43, 43) and data['u_std'].shape == (1, 43, 43)
    for i in range(3):
        a, u = D.darcy_gen(43, np.random.default_rng([7, i]))
        assert np.array_equal(a, data['a'][i])
        assert np.abs(u - data['u'][i]).max() <= 1e-8 * np.abs(u).max()
