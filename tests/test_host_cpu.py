"""CPU-only checks: the C-ABI library loads and exports everything the header declares, host-side helpers agree
with the recorded reference values, argument validation answers before any launch."""
import os
import re

import numpy as np
import torch

from tests.helpers import GOLDEN, ROOT


def test_library_exports_every_declared_symbol():
    import spgt_b200._lib as L
    header = open(os.path.join(ROOT, 'include', 'spgt_b200.h')).read()
    declared = set(re.findall(r'\b(spgt_[a-z0-9_]+)\s*\(', header))
    assert len(declared) >= 23
    for name in sorted(declared):
        assert hasattr(L.lib, name), f'{name} declared in include/spgt_b200.h but not exported'
        assert name in L.SIGNATURES, f'{name} has no ctypes signature'
    assert L.lib.spgt_abi_version() == 1
    assert L.lib.spgt_error_string(-4) == b'workspace missing or too small'


def test_argument_validation_without_gpu():
    from spgt_b200._lib import lib
    assert lib.spgt_batched_transpose(None, None, 4, 4, 1, None) == -1            # NULL
    assert lib.spgt_batched_transpose(16, 32, 0, 4, 1, None) == -2                # bad shape (never dereferenced)
    assert lib.spgt_galerkin_attn_fwd(16, 16, 16, 16, None, 1, 1, 36, 8, 0, None) == -2
    assert lib.spgt_galerkin_attn_fwd(16, 16, 16, 20, None, 1, 1, 34, 8, 0, None) == -3   # misaligned out
    assert lib.spgt_projpos_fwd(16, 16, None, 16, 16, 1, 8, 128, 2, 64, 2, None) == -2    # d_head != 32
    assert lib.spgt_spectral_tables_bytes(211, 12) > 0 and lib.spgt_spectral_tables_bytes(10, 17) == 0
    # Y1 and P [8, 211, 24, 32] + Zr, Zi, Or, Oi [8, 24, 12, 32] + the 2048-float image of the residual weight
    assert lib.spgt_spectral_workspace_bytes(8, 211, 12, 32) == (2 * 8 * 211 * 24 * 32 + 4 * 8 * 24 * 12 * 32 + 2048) * 4
    assert lib.spgt_spectral_launches(8, 211, 12) == 5 and lib.spgt_spectral_chunk_samples(211) >= 8
    assert lib.spgt_skinny_gemm_workspace_bytes(32, 32, 1849, 64) % 4 == 0 and lib.spgt_skinny_gemm_workspace_bytes(32, 30, 1849, 64) % 4096 == 0
    assert lib.spgt_set_tuning(b'no_such_key', 1) == -2


def test_config_and_shapes_match_reference_tables():
    from spgt_b200.common.trivial import get_resolution_size
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import meshgrid
    z = np.load(os.path.join(GOLDEN, 'shapes.npz'))
    for k in z.files:
        a, b = (int(v) for v in k.split('_')[1:])
        if k.startswith('res_'):
            assert np.array_equal(np.array(get_resolution_size(a, b)), z[k]), k
        else:
            assert np.array_equal(meshgrid(a, b), z[k]), k
    cfg = get_darcy_config(2, 8, num_frequence_mode=12)
    assert cfg['r_node'] == 211 and cfg['r_attn'] == 53 and cfg['resolution_size'][1] == (106, 106)
    cfg = get_darcy_config(3, 10, num_frequence_mode=12)
    assert cfg['r_node'] == 141 and cfg['r_attn'] == 43 and cfg['resolution_size'][1] == (77, 77)
    cfg = get_darcy_config()                     # YAML defaults: r_attn 71 stays inside [32, 128]; modes = ceil(sqrt(141))
    assert cfg['r_attn'] == 71 and cfg['num_frequence_mode'] == 12
    cfg = get_darcy_config(1, 2)                 # r_attn 211 is clamped to 128 and subsample_attn recomputed
    assert cfg['r_attn'] == 128 and cfg['subsample_attn'] == 4


def test_model_has_reference_state_dict_keys():
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    z = np.load(os.path.join(GOLDEN, 'model_small.npz'))
    ref_keys = {k[2:]: z[k].shape for k in z.files if k.startswith('p_')}
    cfg = get_darcy_config(3, 6, num_frequence_mode=4, clamp_attn=False, fine_resolution=85, num_encoder_layer=2)
    model = Sp_GalerkinTransformer2D(cfg)
    sd = model.state_dict()
    assert set(sd) == set(ref_keys)
    for k, v in sd.items():
        assert tuple(v.shape) == tuple(ref_keys[k]), k
    full = Sp_GalerkinTransformer2D(get_darcy_config(2, 8, num_frequence_mode=12))
    assert sum(p.numel() for p in full.parameters()) == 2221213


def test_ops_reject_cpu_and_wrong_dtype_tensors():
    import pytest
    from spgt_b200 import ops
    x = torch.randn(1, 8, 128)
    with pytest.raises(ValueError):
        ops.projpos(x, torch.randn(128, 128), None, torch.rand(1, 8, 2), 4, 32, 2)
    with pytest.raises(ValueError):
        ops.batched_transpose(x, [1], [8], [128])
    assert ops.act_code('silu') == 2 and ops.act_code('relu') == 1 and ops.act_code('gelu') == 1 and ops.act_code(None) == 0


def test_synthetic_fields_are_index_deterministic():
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch, GaussNormalizer
    a = synthetic_darcy_batch(range(2, 4), 85, 3, 6, seed=7)
    b = synthetic_darcy_batch(range(0, 4), 85, 3, 6, seed=7)
    assert torch.equal(a['node'], b['node'][2:]) and a['node'].shape == (2, 29, 29, 1)
    assert set(np.unique(a['coeff'].numpy())) <= {3.0, 12.0}
    assert a['position'].shape == (2, 15, 15, 2) and a['grid'].shape == (2, 29, 29, 2)
    n = GaussNormalizer()
    assert float(n.inverse_transform(torch.tensor(2.0))) == 2.0 * (1.0 + 1e-5)


def test_checkpoint_conversion_roundtrip_and_shapes():
    """GT <-> SpGT state dicts: Q/K/V transposed, Fourier weights permuted, everything else untouched; a round trip is exact."""
    import torch
    from spgt_b200.common.checkpoint import gt_to_spgt_state, spgt_to_gt_state
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    torch.manual_seed(0)
    sp = Sp_GalerkinTransformer2D(get_darcy_config(3, 10, num_frequence_mode=12)).state_dict()
    gt = spgt_to_gt_state(sp)
    assert gt.keys() == sp.keys()
    back = gt_to_spgt_state(gt)
    for k in sp:
        assert torch.equal(back[k], sp[k]), k
        last = k.split('.')[-1]
        if last in ('weight_Q', 'weight_K', 'weight_V'):
            assert torch.equal(gt[k], sp[k].t())
        elif 'fourier_weight' in k:
            assert gt[k].shape == (32, 32, 12, 12, 2) and sp[k].shape == (12, 12, 32, 32, 2)
            assert torch.equal(gt[k][3, 5, 7, 2], sp[k][7, 2, 3, 5])
        else:
            assert torch.equal(gt[k], sp[k])


def test_benchmark_weights_fit_the_model_and_the_cpu_baseline():
    """bench.random_state() is a complete state dict of the benchmark model; the CPU baseline of the benchmark (the
    reference's own model when its files are staged, else the restatement) accepts it and both agree with the oracle."""
    import bench
    from oracle import gt_oracle as O, ref_runner as R
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    state = bench.random_state()
    model = Sp_GalerkinTransformer2D(get_darcy_config(2, 8, num_frequence_mode=12))
    model.load_state_dict(state, strict=True)
    # a small shape for the forward check: the same keys minus four encoder layers
    small = {k: v for k, v in bench.random_state(modes=4).items() if not any(f'layers.{i}.attention' in k or f'encoder_mixer.layers.{i}.' in k for i in range(2, 6))}
    ocfg = O.default_config(85, 3, 6, 4, 2, 2)
    data = R.synthetic_batch(range(2), 85, 3, 6, seed=4)
    fwd, kind = R.make_forward(ocfg, small)
    out = fwd(data['node'], data['position'], data['grid'])
    ref = O.model_forward(data['node'], data['position'], data['grid'], small, ocfg)
    assert kind in ('reference', 'port')
    assert float((out - ref).norm() / ref.norm()) < 1e-5
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    mine = synthetic_darcy_batch(range(2), 85, 3, 6, 4)
    assert all(torch.equal(mine[k], data[k]) for k in ('node', 'position', 'grid'))      # both arms see the same samples


def test_weighted_l2_loss_formulas():
    """WeightedL2Loss2D against its definition (and against the reference's class when a checkout is at hand)."""
    from spgt_b200.engine.metric import WeightedL2Loss2D
    g = torch.Generator().manual_seed(4)
    N, r = 3, 11
    pred, target = torch.randn(N, r, r, 1, generator=g), torch.randn(N, r, r, 1, generator=g)
    tgrad, coeff = torch.randn(N, r, r, 2, generator=g), torch.rand(N, r, r, 1, generator=g) + 0.5
    loss, reg, metric = WeightedL2Loss2D(S=r, is_regularization=True, gamma=0.5)(pred, target, None, tgrad, coeff)
    e = ((pred - target) ** 2).mean(dim=[1, 2, 3]) / ((target ** 2).mean(dim=[1, 2, 3]) + 1e-10)
    assert abs(float(loss) - float(e.sqrt().mean())) < 1e-6 and abs(float(metric) - float(e.sqrt().mean())) < 1e-6
    p = pred.squeeze(-1)
    d = torch.stack([(p[:, 2:, 1:-1] - p[:, :-2, 1:-1]) / 2, (p[:, 1:-1, 2:] - p[:, 1:-1, :-2]) / 2], dim=-1) * r
    gn = 2 * (coeff * tgrad ** 2).mean(dim=[1, 2, 3]) + 1e-10
    rr = 0.5 / r * ((coeff[:, 1:-1, 1:-1] * (tgrad[:, 1:-1, 1:-1] - d)) ** 2).mean(dim=[1, 2, 3]) / gn
    assert abs(float(reg) - float(rr.sqrt().mean())) < 1e-6
    l2, r2, m2 = WeightedL2Loss2D(S=r, metric_reduction='L2', is_normalization=False)(pred, target)
    assert abs(float(m2) - float(e.mean().sqrt())) < 1e-6 and abs(float(l2) - float(e.mean())) < 1e-6 and float(r2) == 0.0
    ref_root = os.environ.get('SPGT_REFERENCE', '')
    if os.path.isdir(os.path.join(ref_root, 'engine')):
        from tests.golden.make_golden import import_reference
        import_reference(ref_root)
        from SpGT.engine.metric import WeightedL2Loss2D as Ref
        a = Ref(S=r, is_regularization=True, gamma=0.5)(pred, target, None, tgrad, coeff)
        assert all(abs(float(x) - float(y)) < 1e-6 for x, y in zip(a, (loss, reg, metric)))
