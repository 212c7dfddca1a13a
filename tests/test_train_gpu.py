"""The differentiable (training-mode) forward and the training loop on a B200: gradients against torch autograd through the
float64 CPU oracle, a short training run, and the fused inference path after the weights have changed."""
import numpy as np
import pytest
import torch

from tests.helpers import rel_l2
from oracle import gt_oracle as O

pytestmark = pytest.mark.gpu


def _small():
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import GaussNormalizer, synthetic_darcy_batch
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    cfg = get_darcy_config(3, 6, num_frequence_mode=4, clamp_attn=False, fine_resolution=85, num_encoder_layer=2)
    cfg['target_normalizer'] = GaussNormalizer()
    torch.manual_seed(21)
    model = Sp_GalerkinTransformer2D(cfg)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if 'fourier_weight' in n:
                p.mul_(30.0)
    data = synthetic_darcy_batch(range(2), 85, 3, 6, seed=21)
    return cfg, model, data


def test_training_forward_matches_fused_forward_and_oracle_gradients():
    torch.backends.cudnn.allow_tf32 = False           # the library convolutions of the differentiable path in full fp32
    torch.backends.cuda.matmul.allow_tf32 = False
    cfg, model, data = _small()
    ocfg = O.default_config(85, 3, 6, 4, 2, 2)
    target = torch.randn(2, 29, 29, 1, generator=torch.Generator().manual_seed(3)) * 0.1
    # float64 autograd through the oracle
    p64 = {k: v.detach().double().requires_grad_(True) for k, v in model.state_dict().items()}
    ref = O.model_forward(data['node'].double(), data['position'].double(), data['grid'].double(), p64, ocfg)
    ref_loss = (ref - target.double()).pow(2).mean()
    ref_loss.backward()
    model = model.cuda()
    node, position, grid = (data[k].cuda() for k in ('node', 'position', 'grid'))
    model.train()
    out = model(node, position, grid)
    assert out.requires_grad
    assert rel_l2(out, ref) < 1e-4
    loss = (out - target.cuda()).pow(2).mean()
    loss.backward()
    checked = 0
    for name, prm in model.named_parameters():
        g_ref = p64[name].grad
        if g_ref is None or float(g_ref.norm()) == 0.0:
            continue
        assert prm.grad is not None, name
        assert rel_l2(prm.grad, g_ref) < 1e-3, (name, rel_l2(prm.grad, g_ref))      # fp32 back-propagation through the whole model
        checked += 1
    assert checked >= 40
    model.eval()
    fused = model(node, position, grid)
    assert not fused.requires_grad
    assert rel_l2(fused, out) < 1e-4


def test_short_training_run_reduces_the_loss_and_inference_follows_the_new_weights():
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.run.darcy_train import darcy_train
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    import scipy.ndimage
    rng = np.random.default_rng(5)
    n, R = 8, 85
    a = np.where(scipy.ndimage.gaussian_filter(rng.standard_normal((n, R, R)), [0, 4, 4]) >= 0, 12.0, 3.0).astype(np.float32)
    xx, yy = np.meshgrid(np.linspace(0, 1, R), np.linspace(0, 1, R))
    bump = (np.sin(np.pi * xx) * np.sin(np.pi * yy))[None]
    u = 0.02 * bump * scipy.ndimage.gaussian_filter((a - 7.5) / 4.5, [0, 6, 6])        # a smooth, learnable function of the coefficient
    data = {'a': a, 'u': u.astype(np.float32)}
    cfg = get_darcy_config(3, 6, num_frequence_mode=4, clamp_attn=False, fine_resolution=R, num_encoder_layer=2,
                           num_data=8, batch_size=4, epochs=20, lr=2e-3, seed=7)
    logs = []
    ckpt = darcy_train(cfg, data, data, num_valid=4, log=logs.append)
    assert len(ckpt['loss_history']) == 20 and len(ckpt['metric_history']) == 20, logs
    assert min(ckpt['loss_history'][-3:]) < 0.9 * ckpt['loss_history'][0], ckpt['loss_history']
    assert min(ckpt['metric_history']) < ckpt['metric_history'][0], ckpt['metric_history']
    assert 'Module' in ckpt and ckpt['Best_Metric'] == min(ckpt['metric_history'])
    # the saved state loads into a fresh model whose fused and differentiable paths agree on the trained weights
    from spgt_b200.dataset.darcy_dataset import DarcyDataset
    ds = DarcyDataset(data, 3, 6, 8, R, is_training=True)
    model = Sp_GalerkinTransformer2D(dict(cfg, target_normalizer=ds.target_normalizer.numpy_to_torch('cuda:0')))
    model.load_state_dict(ckpt['Module'])
    model = model.cuda()
    b = next(iter(ds.batches(4)))
    node, position, grid = (b[k].cuda() for k in ('node', 'position', 'grid'))
    model.eval()
    fused = model(node, position, grid)
    model.train()
    with torch.enable_grad():
        diff = model(node, position, grid).detach()
    assert rel_l2(fused, diff) < 1e-4
