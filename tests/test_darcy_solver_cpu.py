"""The oracle of the reference's Darcy data generator (dataset/darcy_generate/*.m), checked by properties: there is no
MATLAB here to generate reference outputs, so its parity is unpinned (see the oracle's header)."""
import numpy as np

from oracle import darcy_solver as D


def test_operator_is_symmetric_positive_definite():
    rng = np.random.default_rng(0)
    a = D.threshold_coefficient(D.gaussian_random_field(29, rng))
    A = D.assemble(D.spline_resample(a, D.centres(29), D.nodes(29)))
    assert abs(A - A.T).max() == 0.0
    assert np.linalg.eigvalsh(A.toarray()).min() > 0.0
    # row sums vanish away from the boundary (pure differences) and are positive next to it
    rs = np.asarray(A.sum(axis=1)).reshape(27, 27)
    assert np.abs(rs[1:-1, 1:-1]).max() < 1e-6 * A.diagonal().max() and rs[0].min() > 0


def test_constant_coefficient_converges_to_the_poisson_series():
    exact = D.poisson_unit_square(0.5, 0.5)
    errs = []
    for K in (17, 33, 65):
        p = D.solve_nodes(np.ones((K, K)), np.ones((K, K)))
        assert p[0].max() == 0 and p[-1].max() == 0 and p[:, 0].max() == 0 and p[:, -1].max() == 0
        errs.append(abs(p[K // 2, K // 2] - exact))
    assert errs[0] > 3.5 * errs[1] > 12 * errs[2]            # second order in the mesh width
    assert errs[2] < 2e-5


def test_solution_satisfies_the_discrete_equations_and_is_positive():
    rng = np.random.default_rng(3)
    a, u = D.darcy_gen(43, rng)
    assert set(np.unique(a)) <= {3.0, 12.0}
    assert u.shape == (43, 43) and u.min() > 0 and 1e-3 < u.max() < 0.1
    cn = D.spline_resample(a, D.centres(43), D.nodes(43))
    fn = D.spline_resample(np.ones((43, 43)), D.centres(43), D.nodes(43))
    p = D.solve_nodes(cn, fn)
    r = D.assemble(cn) @ p[1:-1, 1:-1].ravel() - fn[1:-1, 1:-1].ravel()
    assert np.abs(r).max() < 1e-9
    assert np.allclose(fn, 1.0, atol=1e-12)                  # a spline reproduces the constant forcing


def test_product_host_steps_match_the_oracle():
    """The generator's host-side pieces (random field, resampling) are the same arithmetic as the oracle's."""
    from spgt_b200.dataset import darcy_generate as G
    U1 = D.gaussian_random_field(31, np.random.default_rng([5, 0]))
    U2 = G.gaussian_random_field(31, np.random.default_rng([5, 0]))
    assert np.array_equal(U1, U2)
    Z = np.random.default_rng(1).standard_normal((2, 31, 31))
    assert np.array_equal(G._resample(Z, D.centres(31), D.nodes(31))[1], D.spline_resample(Z[1], D.centres(31), D.nodes(31)))


def test_generated_samples_feed_the_dataset(tmp_path):
    """Samples with the generator's keys (here from the oracle: no GPU) are read by DarcyDataset, from memory and from a
    .mat file written by the generator's writer."""
    from spgt_b200.dataset import darcy_generate as G
    from spgt_b200.dataset.darcy_dataset import DarcyDataset
    pairs = [D.darcy_gen(29, np.random.default_rng([2, i])) for i in range(4)]
    a, u = np.stack([p[0] for p in pairs]), np.stack([p[1] for p in pairs])
    data = {'a': a, 'u': u, 'a_mean': a.mean(0, keepdims=True), 'u_mean': u.mean(0, keepdims=True),
            'a_std': a.std(0, ddof=1, keepdims=True), 'u_std': u.std(0, ddof=1, keepdims=True)}
    ds = DarcyDataset(data, subsample_node=2, subsample_attn=4, num_data=3)
    item = ds[1]
    assert item['node'].shape == (15, 15, 1) and item['target'].shape == (15, 15, 1) and item['position'].shape == (8, 8, 2)
    assert np.allclose(item['target'].numpy()[..., 0], u[1, ::2, ::2], rtol=1e-6)
    G.save_mat(str(tmp_path / 'darcy_R29_N4_1.mat'), data)
    ds2 = DarcyDataset(str(tmp_path / 'darcy_R29_N4_1.mat'), subsample_node=2, subsample_attn=4, num_data=3)
    assert np.array_equal(ds2[1]['node'].numpy(), item['node'].numpy())
