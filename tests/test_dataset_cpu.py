"""The .mat reader and DarcyDataset on a small generated file (scipy v5 format), against the reference's own classes
when the reference checkout is present."""
import os
import sys
import types

import numpy as np
import pytest
import torch

from spgt_b200.dataset.darcy_dataset import DarcyDataset, GaussNormalizer, central_diff, meshgrid
from spgt_b200.dataset.data_accessor import read_matfile

REF = os.environ.get('SPGT_REFERENCE', '')        # location of a checkout of the reference; unset: the live test skips


def _write_mat(path, n=6, R=13, seed=0):
    from scipy.io import savemat
    rng = np.random.default_rng(seed)
    a = np.where(rng.standard_normal((n, R, R)) >= 0, 12.0, 3.0)
    u = rng.standard_normal((n, R, R)) * 0.01
    savemat(path, {'a': a, 'u': u})
    return a.astype(np.float32), u.astype(np.float32)


def test_read_matfile_roundtrip(tmp_path):
    path = str(tmp_path / 'd.mat')
    a, u = _write_mat(path)
    ra, ru = read_matfile(path, ['a', 'u'], [np.float32, np.float64])
    assert ra.dtype == np.float32 and ru.dtype == np.float64
    assert np.array_equal(ra, a) and np.allclose(ru, u)


def test_darcy_dataset_items_and_normalisers(tmp_path):
    path = str(tmp_path / 'd.mat')
    a, u = _write_mat(path, n=6, R=13)
    train = DarcyDataset(path, 3, 6, num_data=4, is_training=True)
    assert len(train) == 4
    it = train[1]
    assert it['node'].shape == (5, 5, 1) and it['grid'].shape == (5, 5, 2) and it['position'].shape == (3, 3, 2)
    assert it['target_grad'].shape == (5, 5, 2) and it['coeff'].dtype == torch.float32
    assert torch.equal(it['coeff'][..., 0], torch.from_numpy(a[1, ::3, ::3]))
    assert torch.equal(it['target'][..., 0], torch.from_numpy(u[1, ::3, ::3]))
    nodes = a[:4, ::3, ::3, None]
    want = (nodes - nodes.mean(0)) / (nodes.std(0) + 1e-5)
    assert np.allclose(it['node'].numpy(), want[1], atol=1e-6)
    gx, gy = central_diff(u, 13)
    assert np.allclose(it['target_grad'][..., 0].numpy(), gx[1, ::3, ::3], atol=1e-6)
    assert np.allclose(it['grid'].numpy(), meshgrid(13, 3), atol=1e-7)
    valid = DarcyDataset(path, 3, 6, num_data=2, is_training=False, node_normalizer=train.node_normalizer)
    assert torch.equal(valid[0]['coeff'][..., 0], torch.from_numpy(a[-2, ::3, ::3]))       # the last samples
    with pytest.raises(ValueError):
        DarcyDataset(path, 3, 6, num_data=2, is_training=False)
    batches = list(train.batches(3))
    assert [b['node'].shape[0] for b in batches] == [3, 1] and batches[0]['position'].shape == (3, 3, 3, 2)


@pytest.mark.skipif(not os.path.isdir(REF), reason='reference checkout not present')
def test_darcy_dataset_matches_reference(tmp_path):
    """Same items as the reference's DarcyDataset on the same file (the reference needs h5py / termcolor only at import)."""
    path = str(tmp_path / 'd.mat')
    _write_mat(path, n=5, R=17, seed=3)
    for name in ('h5py', 'termcolor'):
        if name not in sys.modules:
            try:
                __import__(name)
            except ImportError:
                stub = types.ModuleType(name)
                stub.File = None
                stub.colored = lambda s, *a, **k: s
                sys.modules[name] = stub
    link = tmp_path / 'SpGT'
    os.symlink(REF, link)
    sys.path.insert(0, str(tmp_path))
    try:
        from SpGT.dataset.darcy_dataset import DarcyDataset as RefDataset
        ref_train = RefDataset(path, 2, 4, num_data=3, is_training=True)
        ref_valid = RefDataset(path, 2, 4, num_data=2, is_training=False, node_normalizer=ref_train.node_normalizer)
    finally:
        sys.path.remove(str(tmp_path))
    train = DarcyDataset(path, 2, 4, num_data=3, is_training=True)
    valid = DarcyDataset(path, 2, 4, num_data=2, is_training=False, node_normalizer=train.node_normalizer)
    for mine, ref in ((train, ref_train), (valid, ref_valid)):
        assert len(mine) == len(ref)
        for i in range(len(mine)):
            a, b = mine[i], ref[i]
            assert a.keys() == b.keys()
            for k in a:
                assert torch.allclose(a[k], b[k], atol=1e-6), k
    assert np.allclose(train.target_normalizer.mean, ref_train.target_normalizer.mean, atol=1e-7)
