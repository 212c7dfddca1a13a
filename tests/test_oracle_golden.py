"""The CPU oracle against the fixtures recorded from the reference's own CPU modules."""
import os

import numpy as np
import pytest
import torch

from tests.helpers import GOLDEN, load_golden, rel_l2
from oracle import gt_oracle as O

TOL = 2e-6   # fp32 vs fp32 with a different summation order


def test_resolution_and_meshgrid_tables():
    z = np.load(os.path.join(GOLDEN, 'shapes.npz'))
    for k in z.files:
        a, b = k.split('_')[1:]
        if k.startswith('res_'):
            assert np.array_equal(np.array(O.get_resolution_size(int(a), int(b))), z[k]), k
        else:
            assert np.array_equal(O.meshgrid(int(a), int(b)), z[k]), k
    assert O.get_resolution_size(211, 53)[1] == (106, 106)
    assert O.get_resolution_size(141, 43)[1] == (77, 77)


def test_attention_ops_and_layer():
    d, p = load_golden('attention_layer.npz')
    x, pos = d['x'], d['pos']
    Q = O.projpos(x, p['weight_Q'], p['bias_Q'], pos, 4, 32)
    K = O.projpos_lnorm(x, p['weight_K'], p['bias_K'], p['ln_weight_K'], p['ln_bias_K'], pos, 1e-6, 4, 32)
    V = O.projpos_lnorm(x, p['weight_V'], p['bias_V'], p['ln_weight_V'], p['ln_bias_V'], pos, 1e-6, 4, 32)
    assert rel_l2(Q, d['Q']) < TOL and rel_l2(K, d['K']) < TOL and rel_l2(V, d['V']) < TOL
    assert torch.equal(Q[:, :, :2], d['Q'][:, :, :2])
    assert rel_l2(O.galerkin_attention(d['Q'], d['K'], d['V']), d['attn']) < TOL
    cfg = O.default_config()
    out = O.attention_layer(x, pos, p, '', cfg)
    assert rel_l2(out, d['out']) < TOL


def test_spectral_layer():
    d, p = load_golden('spectral_layer.npz')
    y = O.spectral_conv2d(d['x'], p, '', 4, 'silu')
    assert rel_l2(y, d['y']) < TOL
    y64 = O.spectral_conv2d(d['x'].double(), O.to_dtype(p, torch.float64), '', 4, 'silu')
    assert rel_l2(y64, d['y']) < TOL


def test_datamove_oracles_roundtrip():
    g = torch.Generator().manual_seed(5)
    X = torch.randn(3, 5, 7, 4, generator=g)
    Y = O.batched_transpose(X, [3], [5, 7], [4])
    assert Y.shape == (3, 4, 5, 7) and torch.equal(Y, X.permute(0, 3, 1, 2))
    src = torch.view_as_complex(torch.randn(2, 3, 9, 5, 2, generator=g))
    a, b = O.transpose_gather_dual(src, [2, 3], 9, 5, 4, 3, 0, 0, 5, 0)
    assert a.shape == (4, 3, 2, 3) and torch.equal(a, src[:, :, :4, :3].permute(2, 3, 0, 1))
    assert torch.equal(b, src[:, :, 5:9, :3].permute(2, 3, 0, 1))
    back = O.transpose_scatter_dual(a, b, [2, 3], 9, 5, 4, 3, 0, 0, 5, 0)
    ref = torch.zeros_like(src)
    ref[:, :, :4, :3] = src[:, :, :4, :3]
    ref[:, :, 5:, :3] = src[:, :, 5:, :3]
    assert torch.equal(back, ref)


def test_small_model_taps_and_output():
    d, p = load_golden('model_small.npz')
    cfg = O.default_config(fine_resolution=85, subsample_node=3, subsample_attn=6, num_frequence_mode=4,
                           num_encoder_layer=2, num_decoder_layer=2)
    taps = {}
    out = O.model_forward(d['node'], d['position'], d['grid'], p, cfg, taps)
    for k in ('down', 'enc0', 'enc1', 'up', 'spatial_fc', 'spectral0', 'spectral1', 'decoder'):
        assert rel_l2(taps[k].reshape(-1), d['t_' + k].reshape(-1)) < 5e-6, k
    assert rel_l2(out, d['out']) < 5e-6
    assert float(out[:, 0].abs().max()) == 0.0 and float(out[:, :, -1].abs().max()) == 0.0


REFERENCE = os.environ.get('SPGT_REFERENCE', '')        # location of a checkout of the reference; unset: the live tests skip


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, 'network')), reason='reference checkout not present')
def test_oracle_against_live_reference_attention_config0():
    """BASELINE config 0 (B=4, S=43*43) run through the reference module in this container."""
    from tests.golden.make_golden import import_reference, gt_to_spgt_state
    ref_layer, *_ = import_reference(REFERENCE)
    torch.manual_seed(0)
    attn = ref_layer.GalerkinAttention(128, 4, 2, 1e-6, 0.0, 0.0, 0.01, 0.01, False).eval()
    x = torch.randn(4, 43 * 43, 128)
    pos = torch.from_numpy(O.meshgrid(43, 1)).float().reshape(1, -1, 2).repeat(4, 1, 1)
    with torch.no_grad():
        ref = attn(x, x, x, pos)
    out = O.attention_layer(x, pos, gt_to_spgt_state(attn.state_dict()), '', O.default_config())
    assert rel_l2(out, ref) < TOL
