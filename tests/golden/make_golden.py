"""Generate the golden fixtures in this folder from the reference's own CPU modules.

Run where the reference checkout is available (its location: --reference, or the SPGT_REFERENCE environment
variable):

    python tests/golden/make_golden.py [--reference <reference checkout>]

The reference is imported unmodified as package ``SpGT`` (a temporary directory with a symlink
named SpGT is put on sys.path; ``termcolor`` and ``h5py``, which its support modules import but the
forward never uses, are stubbed).  The pure-PyTorch "GT" modules (network/layer.py,
network/model.py) are run in fp32 on CPU with every drop rate 0, and inputs, weights (converted
to the SpGT op conventions) and outputs are written as .npz files.  Machines that run the GPU tests
need no checkout of the reference: the tests replay these files.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def import_reference(ref_path: str):
    """Expose the read-only reference checkout as package SpGT without writing into it."""
    sys.dont_write_bytecode = True
    tmp = tempfile.mkdtemp(prefix='spgt_ref_')
    os.symlink(ref_path, os.path.join(tmp, 'SpGT'))
    sys.path.insert(0, tmp)
    termcolor = types.ModuleType('termcolor')
    termcolor.colored = lambda s, *a, **k: s
    sys.modules.setdefault('termcolor', termcolor)
    h5py = types.ModuleType('h5py')
    h5py.File = None
    sys.modules.setdefault('h5py', h5py)
    from SpGT.network import layer as ref_layer, model as ref_model
    from SpGT.common.trivial import get_resolution_size
    from SpGT.dataset.darcy_dataset import GaussNormalizer, DarcyDataset
    return ref_layer, ref_model, get_resolution_size, GaussNormalizer, DarcyDataset


from spgt_b200.common.checkpoint import gt_to_spgt_state  # noqa: E402  (GT -> SpGT parameter layouts)


def ref_config(oracle_cfg: dict, normalizer) -> dict:
    cfg = dict(oracle_cfg)
    for k in ('drop_module', 'drop_downscaler', 'drop_upscaler', 'drop_encoder_attn', 'drop_encoder_attn_fc',
              'drop_encoder_ffn', 'drop_decoder_layer'):
        cfg[k] = 0.0
    cfg['target_normalizer'] = normalizer
    return cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', default=os.environ.get('SPGT_REFERENCE'), required='SPGT_REFERENCE' not in os.environ)
    args = ap.parse_args()
    ref_layer, ref_model, ref_get_res, GaussNormalizer, DarcyDataset = import_reference(args.reference)
    from oracle import gt_oracle as O

    torch.set_num_threads(1)      # fixed reduction order for the recorded fp32 values

    # ---- 1. resolution helper and meshgrid: table of known answers -------------------------
    res = {}
    for rl, rs in ((141, 43), (211, 53), (29, 15), (421, 128), (85, 43), (64, 32), (256, 128), (512, 128)):
        res[f'{rl}_{rs}'] = np.array(ref_get_res(rl, rs))
    mesh = {f'{S}_{sub}': DarcyDataset._meshgrid(S, sub, True) for S, sub in ((85, 3), (85, 6), (421, 8))}
    np.savez_compressed(os.path.join(HERE, 'shapes.npz'),
                        **{'res_' + k: v for k, v in res.items()},
                        **{'mesh_' + k: v.astype(np.float64) for k, v in mesh.items()})

    # ---- 2. one Galerkin attention layer ------------------------------------------------------
    torch.manual_seed(0)
    B, ra, D, H = 2, 9, 128, 4
    S = ra * ra
    attn = ref_layer.GalerkinAttention(D, H, 2, 1e-6, 0.0, 0.0, 0.01, 0.01, False).eval()
    # non-trivial LN affine and biases so that they are exercised
    with torch.no_grad():
        for n, prm in attn.named_parameters():
            if n.startswith(('bias_', 'ln_bias')):
                prm.copy_(0.1 * torch.randn_like(prm))
            if n.startswith('ln_weight'):
                prm.copy_(1.0 + 0.1 * torch.randn_like(prm))
    x = torch.randn(B, S, D)
    pos = torch.from_numpy(DarcyDataset._meshgrid(ra, 1, True)).float().reshape(1, S, 2).repeat(B, 1, 1)
    with torch.no_grad():
        Q = attn.multihead_projection_with_position(x, attn.weight_Q, attn.bias_Q, pos, H, 32, 2)
        K = attn.multihead_projection_layernorm_with_position(
            x, attn.weight_K, attn.bias_K, attn.ln_weight_K, attn.ln_bias_K, pos, 1e-6, H, 32, 2)
        V = attn.multihead_projection_layernorm_with_position(
            x, attn.weight_V, attn.bias_V, attn.ln_weight_V, attn.ln_bias_V, pos, 1e-6, H, 32, 2)
        A = attn.multihead_galerkin_attention(Q, K, V, droprate=0.0)
        out = attn(x, x, x, pos)
    sd = gt_to_spgt_state(attn.state_dict())
    np.savez_compressed(
        os.path.join(HERE, 'attention_layer.npz'), x=x.numpy(), pos=pos.numpy(),
        Q=Q.transpose(-2, -1).contiguous().numpy(), K=K.transpose(-2, -1).contiguous().numpy(),
        V=V.transpose(-2, -1).contiguous().numpy(), attn=A.numpy(), out=out.numpy(),
        **{'p_' + k: v.numpy() for k, v in sd.items()})

    # ---- 3. one spectral layer -----------------------------------------------------------------
    torch.manual_seed(3)
    N, r, C, m = 2, 19, 32, 4
    spec = ref_layer.SpectralConv2D(C, C, m, 0.0, 'silu').eval()
    with torch.no_grad():   # scale the fourier weights up so the spectral branch is not negligible
        for prm in spec.fourier_weight:
            prm.mul_(30.0)
    xs = torch.randn(N, r, r, C)
    with torch.no_grad():
        ys = spec(xs)
    sd = gt_to_spgt_state(spec.state_dict())
    np.savez_compressed(os.path.join(HERE, 'spectral_layer.npz'), x=xs.numpy(), y=ys.numpy(),
                        **{'p_' + k: v.numpy() for k, v in sd.items()})

    # ---- 4. a small full model -------------------------------------------------------------------
    torch.manual_seed(1)
    ocfg = O.default_config(fine_resolution=85, subsample_node=3, subsample_attn=6, num_frequence_mode=4,
                            num_encoder_layer=2, num_decoder_layer=2)
    assert tuple(map(tuple, ref_get_res(ocfg['r'], ocfg['r_attn']))) == ocfg['resolution_size']
    model = ref_model.GalerkinTransformer2D(ref_config(ocfg, GaussNormalizer())).eval()
    with torch.no_grad():
        for n, prm in model.named_parameters():
            if 'fourier_weight' in n:
                prm.mul_(30.0)
    n_s = 1
    a = O.darcy_coefficient(n_s, 85, 3, seed=1)
    node = torch.from_numpy((a - a.mean()) / (a.std() + 1e-5)).float()
    position = torch.from_numpy(DarcyDataset._meshgrid(85, 6, True)).float().unsqueeze(0).repeat(n_s, 1, 1, 1)
    grid = torch.from_numpy(DarcyDataset._meshgrid(85, 3, True)).float().unsqueeze(0).repeat(n_s, 1, 1, 1)
    taps = {}
    with torch.no_grad():
        xd = model.down_scaler(node)
        taps['down'] = xd
        xe = xd.view(n_s, -1, 128)
        for i, layer in enumerate(model.encoder_mixer.layers):
            xe = layer(xe, position.view(n_s, -1, 2))
            taps[f'enc{i}'] = xe
        xu = model.up_scaler(xe.view(n_s, ocfg['r_attn'], ocfg['r_attn'], 128))
        taps['up'] = xu
        dec = model.decoder_regressor
        xs_ = dec.spatial_fc_layer(torch.concat([xu, grid], dim=-1))
        taps['spatial_fc'] = xs_
        for i, layer in enumerate(dec.layers):
            xs_ = layer(xs_)
            taps[f'spectral{i}'] = xs_
        taps['decoder'] = dec.ffn_layer(xs_)
        out = model(node, position, grid)
    sd = gt_to_spgt_state(model.state_dict())
    np.savez_compressed(
        os.path.join(HERE, 'model_small.npz'), node=node.numpy(), position=position.numpy(), grid=grid.numpy(),
        out=out.numpy(), **{'t_' + k: v.numpy() for k, v in taps.items()},
        **{'p_' + k: v.numpy() for k, v in sd.items()})
    for f in sorted(os.listdir(HERE)):
        if f.endswith('.npz'):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, 'KiB')


if __name__ == '__main__':
    main()
