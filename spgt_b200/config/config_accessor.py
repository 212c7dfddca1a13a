"""Darcy hyper-parameters (reference: config/darcy_config.yaml, config/config_accessor.py:15-40) as a plain dict."""
import math

from ..common.trivial import get_resolution_size

DARCY_DEFAULTS = dict(
    num_data=1024, dim_node=1, dim_target=1, dim_position=2, noise=0.0, boundary_condition='dirichlet',
    fine_resolution=421, subsample_node=3, subsample_attn=6,
    name_module='SpGT', dim_hidden=128, drop_module=0.0,
    drop_downscaler=0.05, acti_downscaler='relu', drop_upscaler=0.0, acti_upscaler='silu', resolution_size=None,
    num_encoder_layer=6, num_head=4, attn_xavier=0.01, attn_diagonal=0.01, attn_symmetric=False, attn_norm_eps=1.0e-6,
    drop_encoder_attn=0.0, drop_encoder_attn_fc=0.05, dim_encoder_ffn=256, drop_encoder_ffn=0.05, acti_encoder_ffn='relu',
    num_decoder_layer=2, drop_decoder_layer=0.0, acti_decoder_layer='silu', dim_spatial_hidden=32, num_frequence_mode=12,
    seed=1127802, metric_gamma=0.5, lr=1.0e-3, epochs=100, batch_size=4, num_load_worker=8,
)


def get_darcy_config(sub_node=None, sub_attn=None, num_frequence_mode=None, clamp_attn=True, **overrides) -> dict:
    """The reference's post-processing of the YAML: r_node and r_attn from the sub-sampling factors, r_attn clamped
    to [32, 128] with subsample_attn recomputed, resolution_size derived, and num_frequence_mode = ceil(sqrt(r_node))
    unless given explicitly.  clamp_attn=False keeps the requested subsample_attn (small test grids)."""
    cfg = dict(DARCY_DEFAULTS)
    cfg.update(overrides)
    if sub_node is not None:
        cfg['subsample_node'] = sub_node
        cfg['subsample_attn'] = sub_attn if sub_attn is not None else sub_node * 2
    R = cfg['fine_resolution']
    r_node = int((R - 1) / cfg['subsample_node'] + 1)
    r_attn = int((R - 1) / cfg['subsample_attn'] + 1)
    if clamp_attn:
        r_attn = max(32, min(128, r_attn))
        cfg['subsample_attn'] = int((R - 1) / r_attn + 1)
    cfg['r_node'], cfg['r_attn'] = r_node, r_attn
    cfg['resolution_size'] = get_resolution_size(r_node, r_attn)
    cfg['num_frequence_mode'] = num_frequence_mode if num_frequence_mode is not None else math.ceil(math.sqrt(r_node))
    return cfg
