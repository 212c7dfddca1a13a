"""Layer- and model-level parity on a B200: recorded reference outputs (tests/golden) and the CPU oracle."""
import pytest
import torch

from tests.helpers import load_golden, rel_l2
from oracle import gt_oracle as O

pytestmark = pytest.mark.gpu
PER_LAYER_TOL = 1e-5     # relative L2 per layer
MODEL_TOL = 1e-4         # relative L2 at the model output


def small_cfg():
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import GaussNormalizer
    cfg = get_darcy_config(3, 6, num_frequence_mode=4, clamp_attn=False, fine_resolution=85, num_encoder_layer=2)
    cfg['target_normalizer'] = GaussNormalizer()
    return cfg


def test_attention_layer_against_golden():
    from spgt_b200.network.sp_layer import Sp_GalerkinAttention
    d, p = load_golden('attention_layer.npz')
    layer = Sp_GalerkinAttention(128, 4, 2, 1e-6, 0.0, 0.0, 0.01, 0.01, False)
    layer.load_state_dict(p)
    layer = layer.cuda()
    x, pos = d['x'].cuda(), d['pos'].cuda()
    with torch.no_grad():
        out = layer(x, x, x, pos)
        out2 = layer(x, x.clone(), x.clone(), pos)       # separate-launch path
    assert rel_l2(out, d['out']) < PER_LAYER_TOL
    assert rel_l2(out2, d['out']) < PER_LAYER_TOL       # different projection kernels, same tolerance


def test_spectral_layer_both_structures():
    from spgt_b200.network.sp_layer import Sp_SpectralConv2D
    d, p = load_golden('spectral_layer.npz')
    for structure in ('fused', 'reference'):
        layer = Sp_SpectralConv2D(32, 32, 4, 0.0, 'silu', structure=structure)
        layer.load_state_dict(p)
        layer = layer.cuda()
        with torch.no_grad():
            y = layer(d['x'].cuda())
        assert rel_l2(y, d['y']) < PER_LAYER_TOL, structure


def test_small_model_against_golden():
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    d, p = load_golden('model_small.npz')
    model = Sp_GalerkinTransformer2D(small_cfg())
    missing = model.load_state_dict(p, strict=True)
    model = model.cuda().eval()
    node, position, grid = d['node'].cuda(), d['position'].cuda(), d['grid'].cuda()
    taps = {}
    out = model(node, position, grid, taps)
    assert rel_l2(taps['down'], d['t_down']) < PER_LAYER_TOL
    assert rel_l2(taps['enc0'].reshape(-1), d['t_enc0'].reshape(-1)) < PER_LAYER_TOL
    assert rel_l2(taps['enc1'].reshape(-1), d['t_enc1'].reshape(-1)) < 2 * PER_LAYER_TOL      # two layers deep
    with torch.no_grad():
        up = model.up_scaler(d['t_enc1'].reshape(1, 15, 15, 128).cuda())
        dec = model.decoder_regressor(d['t_up'].cuda(), grid)
        dec_fused = model.decoder_regressor.forward_from_mid(
            model.up_scaler.forward_mid(d['t_enc1'].reshape(1, 15, 15, 128).cuda()), grid, 1.0, 0.0, False)
    assert rel_l2(up, d['t_up']) < PER_LAYER_TOL
    assert rel_l2(dec, d['t_decoder']) < 3 * PER_LAYER_TOL            # fc + two spectral layers + head
    assert rel_l2(dec_fused, d['t_decoder']) < 3 * PER_LAYER_TOL
    assert rel_l2(out, d['out']) < MODEL_TOL
    assert float(out[:, 0].abs().max()) == 0.0 and float(out[:, :, -1].abs().max()) == 0.0
    assert torch.equal(out, model(node, position, grid))                 # bitwise reproducible


@pytest.mark.parametrize('sub_node,sub_attn,batch', [(3, 10, 2), (2, 8, 1)])
def test_full_size_model_against_oracle(sub_node, sub_attn, batch):
    """BASELINE configs 1 (141^2/43^2) and 4 (211^2/53^2) with random-init weights, vs the fp32 CPU oracle."""
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import GaussNormalizer, synthetic_darcy_batch
    cfg = get_darcy_config(sub_node, sub_attn, num_frequence_mode=12)
    cfg['target_normalizer'] = GaussNormalizer()
    torch.manual_seed(sub_node)
    model = Sp_GalerkinTransformer2D(cfg).eval()
    with torch.no_grad():
        for n, prm in model.named_parameters():
            if 'fourier_weight' in n:
                prm.mul_(30.0)          # make the spectral branch contribute visibly
    data = synthetic_darcy_batch(range(batch), 421, sub_node, cfg['subsample_attn'], seed=sub_node)
    ocfg = O.default_config(421, sub_node, cfg['subsample_attn'], 12)
    assert tuple(ocfg['resolution_size']) == tuple(cfg['resolution_size'])
    p = {k: v.detach().clone() for k, v in model.state_dict().items()}
    ref_taps = {}
    torch.set_num_threads(max(1, torch.get_num_threads()))
    ref = O.model_forward(data['node'], data['position'], data['grid'], p, ocfg, ref_taps)
    model = model.cuda()
    taps = {}
    out = model(data['node'].cuda(), data['position'].cuda(), data['grid'].cuda(), taps)
    assert rel_l2(taps['down'], ref_taps['down']) < PER_LAYER_TOL
    for i in range(6):
        assert rel_l2(taps[f'enc{i}'].reshape(-1), ref_taps[f'enc{i}'].reshape(-1)) < (i + 1) * PER_LAYER_TOL, i
    assert rel_l2(out, ref) < MODEL_TOL


def _random_model(sub_node, sub_attn, modes, seed):
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import GaussNormalizer
    cfg = get_darcy_config(sub_node, sub_attn, num_frequence_mode=modes, clamp_attn=False)
    cfg['target_normalizer'] = GaussNormalizer()
    torch.manual_seed(seed)
    model = Sp_GalerkinTransformer2D(cfg).eval()
    with torch.no_grad():
        for n, prm in model.named_parameters():
            if 'fourier_weight' in n:
                prm.mul_(30.0)
    return cfg, model


def test_super_resolution_shape_against_oracle():
    """Full resolution r = 421 (the reference's super-resolution evaluation grid), attention grid 106^2 = 11236 nodes,
    15 Fourier modes, batch 1, vs the fp32 CPU oracle."""
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    cfg, model = _random_model(1, 4, 15, seed=11)
    data = synthetic_darcy_batch(range(1), 421, 1, 4, seed=11)
    ocfg = O.default_config(421, 1, 4, 15)
    assert tuple(ocfg['resolution_size']) == tuple(cfg['resolution_size'])
    p = {k: v.detach().clone() for k, v in model.state_dict().items()}
    ref = O.model_forward(data['node'], data['position'], data['grid'], p, ocfg)
    out = model.cuda()(data['node'].cuda(), data['position'].cuda(), data['grid'].cuda())
    assert out.shape == (1, 421, 421, 1)
    assert rel_l2(out, ref) < MODEL_TOL


def test_graph_captured_forward_is_bit_identical():
    """A forward captured into a CUDA graph replays to exactly the eager result, also for new inputs."""
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    from spgt_b200.engine.darcy_engine import GraphedForward
    cfg, model = _random_model(3, 10, 12, seed=5)
    model = model.cuda()
    a = {k: v.cuda() for k, v in synthetic_darcy_batch(range(2), 421, 3, 10, seed=5).items()}
    b = {k: v.cuda() for k, v in synthetic_darcy_batch(range(2, 4), 421, 3, 10, seed=5).items()}
    with torch.no_grad():
        eager_a = model(a['node'], a['position'], a['grid']).clone()
        eager_b = model(b['node'], b['position'], b['grid']).clone()
        graphed = GraphedForward(model, a['node'], a['position'], a['grid'])
        assert torch.equal(graphed(a['node']), eager_a)
        assert torch.equal(graphed(b['node'], b['position'], b['grid']), eager_b)
        assert torch.equal(graphed(a['node']), eager_a)
    with pytest.raises(ValueError):
        graphed(a['node'][:1])


def test_host_inference_with_and_without_graphs_agree():
    """The host-facing loop (pinned batches in, pinned predictions out) gives the same bits eagerly and with replayed graphs,
    and every one of its returned predictions - more batches than it has staging slots or ever had output buffers - is the
    prediction of its own batch."""
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    from spgt_b200.engine.darcy_engine import HostInference
    cfg, model = _random_model(3, 10, 12, seed=6)
    model = model.cuda()
    batches = []
    for i in range(7):
        d = synthetic_darcy_batch(range(2 * i, 2 * i + 2), 421, 3, 10, seed=6)
        batches.append({k: d[k].pin_memory() for k in ('node', 'position', 'grid')})
    with torch.no_grad():
        eager = HostInference(model, 'cuda:0').run(batches)
        graphed = HostInference(model, 'cuda:0', use_graphs=True).run(batches)
        direct = [model(b['node'].cuda(), b['position'].cuda(), b['grid'].cuda()).cpu() for b in batches]
    assert len(eager) == len(graphed) == 7
    assert len({t.data_ptr() for t in eager}) == 7            # one host tensor per batch: no prediction overwrites another
    for a, b, c in zip(eager, graphed, direct):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_host_inference_static_inputs_are_uploaded_once_and_refreshed_when_they_change():
    """static_keys: node coordinates that stay the same host tensors are not copied again, new tensors are."""
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    from spgt_b200.engine.darcy_engine import HostInference
    cfg, model = _random_model(3, 10, 12, seed=7)
    model = model.cuda()
    d = synthetic_darcy_batch(range(8), 421, 3, 10, seed=7)
    pos, grid = d['position'][:2].contiguous().pin_memory(), d['grid'][:2].contiguous().pin_memory()
    batches = [{'node': d['node'][2 * i:2 * i + 2].contiguous().pin_memory(), 'position': pos, 'grid': grid} for i in range(4)]
    eng = HostInference(model, 'cuda:0', use_graphs=True, static_keys=('position', 'grid'))
    assert eng.bytes_per_batch(batches[0])['h2d'] == batches[0]['node'].numel() * 4
    with torch.no_grad():
        got = [t.clone() for t in eng.run(batches)]
        direct = [model(b['node'].cuda(), pos.cuda(), grid.cuda()).cpu() for b in batches]
        for a, c in zip(got, direct):
            assert torch.equal(a, c)
        grid2 = (grid * 0.5).pin_memory()                      # another discretisation: must reach the device
        got2 = eng.run([dict(b, grid=grid2) for b in batches])
        direct2 = [model(b['node'].cuda(), pos.cuda(), grid2.cuda()).cpu() for b in batches]
        for a, c in zip(got2, direct2):
            assert torch.equal(a, c)
        assert not torch.equal(got2[0], got[0])
        grid2.mul_(2.0)                                        # changed in place: the version counter tells
        got3 = eng.run([dict(b, grid=grid2) for b in batches])
        for a, c in zip(got3, direct):
            assert torch.equal(a, c)


def test_real_data_inference_driver(tmp_path):
    """run/darcy_inference.py on a small generated .mat file with a saved checkpoint: metric vs the CPU oracle."""
    import numpy as np
    from scipy.io import savemat
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import DarcyDataset
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    from spgt_b200.run.darcy_inference import darcy_inference
    R, n = 85, 15
    rng = np.random.default_rng(8)
    a = np.where(rng.standard_normal((n, R, R)) >= 0, 12.0, 3.0)
    u = rng.standard_normal((n, R, R)) * 0.01
    path = str(tmp_path / 'darcy_small.mat')
    savemat(path, {'a': a, 'u': u})
    cfg = get_darcy_config(3, 6, num_frequence_mode=4, clamp_attn=False, fine_resolution=R, batch_size=1, num_data=13)
    torch.manual_seed(3)
    ckpt = {'Module': Sp_GalerkinTransformer2D(dict(cfg, target_normalizer=None)).state_dict()}
    torch.save(ckpt, str(tmp_path / 'm.pt'))
    ckpt = torch.load(str(tmp_path / 'm.pt'), map_location='cpu')
    metric = darcy_inference(cfg, ckpt, path, path, use_graphs=True)
    # oracle: same normalisers, same batches of 2, mean over batches of the per-batch mean relative L2
    train = DarcyDataset(path, 3, is_training=True)
    valid = DarcyDataset(path, 3, 6, 13, R, is_training=False, node_normalizer=train.node_normalizer)
    ocfg = O.default_config(R, 3, 6, 4)
    ocfg['target_std'] = torch.from_numpy(np.asarray(train.target_normalizer.std)).float()
    ocfg['target_mean'] = torch.from_numpy(np.asarray(train.target_normalizer.mean)).float()
    total, nb = 0.0, 0
    for b in valid.batches(2):
        pred = O.model_forward(b['node'], b['position'], b['grid'], ckpt['Module'], ocfg)
        total += float(O.relative_l2_metric(pred, b['target']))
        nb += 1
    assert nb == 7          # six full batches (more than the host loop has staging slots) and a ragged one
    assert abs(metric - total / nb) < 1e-4 * (total / nb)
