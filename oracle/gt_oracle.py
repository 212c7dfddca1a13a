"""CPU oracle for the SpGT inference hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch CPU tensor math, what the reference's
pure-PyTorch "GT" twin computes for every step of the accelerated SpGT forward
(reference files network/layer.py and network/model.py), re-expressed in the
tensor layouts and weight conventions of the SpGT custom ops
(extension/bind/galerkin_attention.py, extension/bind/datamove.py).  It is the
checker for the CUDA kernels: only the tests, the smoke check and the
benchmark's CPU-baseline leg may import it.  The product package never does.

Parity status: the reference ships no golden vectors or known-answer tests for
this path, so the oracle is pinned against outputs of the reference's own CPU
modules, generated where a checkout of the reference is at hand (tests/golden/make_golden.py writes
them to tests/golden/*.npz; tests/test_oracle_golden.py replays them).

Conventions that differ between the reference's GT modules and its SpGT ops,
and which this oracle applies:
  * SpGT projection ops compute x @ W (the kernel indexes W as [k][n],
    extension/native/multihead_dim32.cu:344), GT computes F.linear(x, W) = x @ W.T
    (network/layer.py:107).  Oracle functions take the SpGT weight.
  * SpGT Q/K/V are [B, H, d_pos + d_head, S] (sequence fastest); GT uses
    [B, H, S, d_pos + d_head] (network/layer.py:108-112).
  * SpGT fourier weights are [m, m, in, out, 2] (network/sp_layer.py:119-121);
    GT uses [in, out, m, m, 2] (network/layer.py:214-216).
  * Every dropout rate is 0: the reference calls F.dropout with training=True
    even in eval mode (e.g. network/sp_layer.py:76), which no deterministic
    implementation can match.

All functions take a dtype so that the same code gives the fp32 result (what
the reference CPU path produces) and an fp64 ground truth for error budgeting.
"""
from __future__ import annotations

import math
from typing import Dict, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# ----------------------------------------------------------------------------
# shape helpers
# ----------------------------------------------------------------------------
def get_resolution_size(r_large: int, r_small: int):
    """Resolutions after each of the four interpolations.

    Follows common/trivial.py:78-96 (round the scale factor sqrt(r_small/r_large)
    to a multiple of 0.005 with a digit-dependent nudge, r_mid = round(r*f) - 1).
    """
    factor = round(float(np.sqrt(r_small / r_large)), ndigits=4)
    last_digit = float(str(factor)[-1])
    factor = round(factor, ndigits=3)
    if last_digit < 5:
        factor += 5.0e-3
    factor = int(factor / 5.0e-3 + 0.5) * 5.0e-3
    r_mid = round(r_large * factor) - 1
    return ((r_large, r_large), (r_mid, r_mid), (r_small, r_small), (r_mid, r_mid), (r_large, r_large))


def meshgrid(S: int, sub: int) -> np.ndarray:
    """Node coordinates of the sub-sampled unit square, [r, r, 2] (x then y).

    Follows dataset/darcy_dataset.py:117-127 with is_return_boundary=True.
    """
    x, y = np.meshgrid(np.linspace(0, 1, S), np.linspace(0, 1, S))
    return np.stack([x[::sub, ::sub], y[::sub, ::sub]], axis=-1)


# ----------------------------------------------------------------------------
# op-level oracles (SpGT layouts)
# ----------------------------------------------------------------------------
def projpos(x: Tensor, weight: Tensor, bias: Tensor, position: Tensor, num_head: int, dim_head: int) -> Tensor:
    """multihead_projection_with_position_rrc: out[b,h,2+c,s] = (x @ W + bias)[b,s,32h+c]; rows 0,1 = position.

    GT definition: network/layer.py:96-113; SpGT op: extension/bind/galerkin_attention.cu:9-24.
    """
    B, S, D = x.shape
    y = x @ weight + bias                                   # [B,S,D]
    y = y.view(B, S, num_head, dim_head).permute(0, 2, 3, 1)  # [B,H,d,S]
    pos = position.transpose(1, 2).unsqueeze(1).expand(B, num_head, position.shape[-1], S)
    return torch.cat([pos, y], dim=2).contiguous()


def projpos_lnorm(
    x: Tensor, weight: Tensor, bias: Tensor, ln_weight: Tensor, ln_bias: Tensor, position: Tensor,
    norm_eps: float, num_head: int, dim_head: int, return_invsigma: bool = False,
):
    """multihead_projection_layernorm_with_position_rrc.

    Per (b, s, h): biased variance over the 32 head channels, y = (v - mu) * rsqrt(var + eps) * lnw[h] + lnb[h];
    position rows are not normalised.  GT definition: network/layer.py:115-142 (F.layer_norm per head);
    SpGT op: extension/bind/galerkin_attention.cu:50-68, LayerNorm math extension/native/multihead_dim32.cu:59-146.
    """
    B, S, D = x.shape
    y = (x @ weight + bias).view(B, S, num_head, dim_head)
    mu = y.mean(dim=-1, keepdim=True)
    var = ((y - mu) ** 2).mean(dim=-1, keepdim=True)
    invsigma = torch.rsqrt(var + norm_eps)
    y = (y - mu) * invsigma * ln_weight.view(1, 1, num_head, dim_head) + ln_bias.view(1, 1, num_head, dim_head)
    y = y.permute(0, 2, 3, 1)
    pos = position.transpose(1, 2).unsqueeze(1).expand(B, num_head, position.shape[-1], S)
    out = torch.cat([pos, y], dim=2).contiguous()
    if return_invsigma:
        return out, invsigma.squeeze(-1).permute(0, 2, 1).contiguous()   # [B,H,S]
    return out


def galerkin_kv(K: Tensor, V: Tensor) -> Tensor:
    """T[b,h,i,j] = (1/S) * sum_s K[b,h,i,s] * V[b,h,j,s]  (network/layer.py:149)."""
    S = K.shape[-1]
    return (K @ V.transpose(-2, -1)) / S


def galerkin_attention(Q: Tensor, K: Tensor, V: Tensor) -> Tensor:
    """multihead_galerkin_attention_cccr: Q,K,V [B,H,dpk,S] -> [B,H,S,dpk], out = Q^T (K V^T / S).

    GT definition: network/layer.py:144-152; SpGT op: extension/bind/galerkin_attention.cu:104-124.
    """
    T = galerkin_kv(K, V)
    return (Q.transpose(-2, -1) @ T).contiguous()


def batched_skinny_gemm(A: Tensor, B: Tensor, alpha: float = 1.0) -> Tensor:
    """C[..., M, N] = alpha * A[..., M, K] @ B[..., K, N]  (extension/bind/galerkin_attention.cu:175-198)."""
    return alpha * (A @ B)


def batched_transpose(X: Tensor, batch_list: Sequence[int], M_list: Sequence[int], N_list: Sequence[int]) -> Tensor:
    """[prod(batch), prod(M), prod(N)] -> shape batch + N + M  (extension/bind/datamove.cu:8-23)."""
    b, M, N = int(np.prod(batch_list)), int(np.prod(M_list)), int(np.prod(N_list))
    out = X.reshape(b, M, N).transpose(1, 2).contiguous()
    return out.view(*batch_list, *N_list, *M_list)


def transpose_gather_dual(
    src: Tensor, dim_list: Sequence[int], H_all: int, W_all: int, H_low: int, W_low: int,
    H_base_1: int, W_base_1: int, H_base_2: int, W_base_2: int,
) -> Tuple[Tensor, Tensor]:
    """Two corner blocks of a complex [dim..., H_all, W_all] tensor, each moved to [H_low, W_low, dim...].

    extension/bind/datamove.cu:25-44, index map extension/native/datamove.cu:34-61.
    """
    dim = int(np.prod(dim_list))
    s = src.reshape(dim, H_all, W_all)
    outs = []
    for hb, wb in ((H_base_1, W_base_1), (H_base_2, W_base_2)):
        blk = s[:, hb:hb + H_low, wb:wb + W_low].permute(1, 2, 0).contiguous()
        outs.append(blk.view(H_low, W_low, *dim_list))
    return outs[0], outs[1]


def transpose_scatter_dual(
    src1: Tensor, src2: Tensor, dim_list: Sequence[int], H_all: int, W_all: int, H_low: int, W_low: int,
    H_base_1: int, W_base_1: int, H_base_2: int, W_base_2: int,
) -> Tensor:
    """Inverse of transpose_gather_dual into a zero-filled [dim..., H_all, W_all] complex tensor.

    extension/bind/datamove.cu:46-64 (torch::zeros output), extension/native/datamove.cu:63-89.
    """
    dim = int(np.prod(dim_list))
    out = torch.zeros(dim, H_all, W_all, dtype=src1.dtype)
    for src, hb, wb in ((src1, H_base_1, W_base_1), (src2, H_base_2, W_base_2)):
        out[:, hb:hb + H_low, wb:wb + W_low] = src.reshape(H_low, W_low, dim).permute(2, 0, 1)
    return out.view(*dim_list, H_all, W_all)


# ----------------------------------------------------------------------------
# layer-level oracles
# ----------------------------------------------------------------------------
def _act(name: str):
    # network/layer.py:14,163: only 'silu' selects SiLU, anything else is ReLU.
    return F.silu if name == 'silu' else F.relu


def feed_forward(x: Tensor, p: Dict[str, Tensor], prefix: str, activation: str) -> Tensor:
    """Linear -> activation -> Linear  (network/layer.py:155-174, dropout rate 0)."""
    h = _act(activation)(F.linear(x, p[prefix + 'layer1.weight'], p[prefix + 'layer1.bias']))
    return F.linear(h, p[prefix + 'layer2.weight'], p[prefix + 'layer2.bias'])


def attention_layer(x: Tensor, position: Tensor, p: Dict[str, Tensor], prefix: str, cfg: dict, taps: dict = None) -> Tensor:
    """Sp_GalerkinAttention.forward with Q=K=V=x  (network/sp_layer.py:52-78)."""
    H, d = cfg['num_head'], cfg['dim_hidden'] // cfg['num_head']
    eps = cfg['attn_norm_eps']
    B, S, D = x.shape
    Q = projpos(x, p[prefix + 'weight_Q'], p[prefix + 'bias_Q'], position, H, d)
    K = projpos_lnorm(x, p[prefix + 'weight_K'], p[prefix + 'bias_K'], p[prefix + 'ln_weight_K'],
                      p[prefix + 'ln_bias_K'], position, eps, H, d)
    V = projpos_lnorm(x, p[prefix + 'weight_V'], p[prefix + 'bias_V'], p[prefix + 'ln_weight_V'],
                      p[prefix + 'ln_bias_V'], position, eps, H, d)
    A = galerkin_attention(Q, K, V)                         # [B,H,S,dpk]
    merged = A.transpose(1, 2).contiguous().view(B, S, H * A.shape[-1])
    out = F.linear(merged, p[prefix + 'fc_layer.weight'], p[prefix + 'fc_layer.bias'])
    if taps is not None:
        taps.update(Q=Q, K=K, V=V, T=galerkin_kv(K, V), attn=A, fc=out)
    return out


def encoder_layer(x: Tensor, position: Tensor, p: Dict[str, Tensor], prefix: str, cfg: dict, taps: dict = None) -> Tensor:
    """Sp_EncoderLayer.forward (network/sp_layer.py:94-104)."""
    x = x + attention_layer(x, position, p, prefix + 'attention_layer.', cfg, taps)
    if taps is not None:
        taps['post_attn'] = x
    x = x + feed_forward(x, p, prefix + 'ffn_layer.', cfg['acti_encoder_ffn'])
    return x


def spectral_conv2d(x: Tensor, p: Dict[str, Tensor], prefix: str, mode: int, activation: str) -> Tensor:
    """Sp_SpectralConv2D.forward  (network/sp_layer.py:125-156; GT twin network/layer.py:219-246).

    x [N, r, r, Cin]; fourier weights in the SpGT layout [m, m, Cin, Cout, 2].
    """
    N, r, _, cin = x.shape
    m = mode
    res = F.linear(x, p[prefix + 'residual_layer.weight'], p[prefix + 'residual_layer.bias'])
    xt = x.permute(0, 3, 1, 2)
    x_ft = torch.fft.rfft2(xt, s=(r, r), norm='ortho')                     # [N,Cin,r,r//2+1]
    w0 = torch.view_as_complex(p[prefix + 'fourier_weight.0'].contiguous())  # [m,m,Cin,Cout]
    w1 = torch.view_as_complex(p[prefix + 'fourier_weight.1'].contiguous())
    cout = w0.shape[-1]
    out_ft = torch.zeros(N, cout, r, r // 2 + 1, dtype=x_ft.dtype)
    out_ft[:, :, :m, :m] = torch.einsum('nihw,hwio->nohw', x_ft[:, :, :m, :m], w0)
    out_ft[:, :, r - m:, :m] = torch.einsum('nihw,hwio->nohw', x_ft[:, :, r - m:, :m], w1)
    y = torch.fft.irfft2(out_ft, s=(r, r), norm='ortho').permute(0, 2, 3, 1)
    return _act(activation)(y + res)


def down_scaler(x: Tensor, p: Dict[str, Tensor], cfg: dict) -> Tensor:
    """DownScaler2D.forward (network/model.py:23-39): [N,r,r,1] -> [N,r_attn,r_attn,D].

    Each ConvResBlock2D already ends in the activation (network/layer.py:21-23); the extra activation after
    conv0's interpolation (network/model.py:31) and after the final interpolation (:37) are kept as written.
    """
    act = _act(cfg['acti_downscaler'])
    rs = cfg['resolution_size']
    pre = 'down_scaler.'
    x = x.permute(0, 3, 1, 2)
    x = act(F.conv2d(x, p[pre + 'conv0.conv_layer.weight'], p[pre + 'conv0.conv_layer.bias'], padding=1))
    x = act(F.interpolate(x, size=rs[1], mode='bilinear', align_corners=True))
    x1 = act(F.conv2d(x, p[pre + 'conv1.conv_layer.weight'], p[pre + 'conv1.conv_layer.bias'], padding=1))
    x2 = act(F.conv2d(x1, p[pre + 'conv2.conv_layer.weight'], p[pre + 'conv2.conv_layer.bias'], padding=1))
    x3 = act(F.conv2d(x2, p[pre + 'conv3.conv_layer.weight'], p[pre + 'conv3.conv_layer.bias'], padding=1))
    x = torch.cat([x1, x2, x3], dim=1)
    x = act(F.interpolate(x, size=rs[2], mode='bilinear', align_corners=True))
    return x.permute(0, 2, 3, 1).contiguous()


def up_scaler(x: Tensor, p: Dict[str, Tensor], cfg: dict) -> Tensor:
    """UpScaler2D.forward (network/model.py:53-65): [N,r_attn,r_attn,D] -> [N,r,r,D]."""
    act = _act(cfg['acti_upscaler'])
    rs = cfg['resolution_size']
    x = x.permute(0, 3, 1, 2)
    x = F.interpolate(x, size=rs[3], mode='bilinear', align_corners=True)
    # The activation is applied twice: once inside ConvResBlock2D.forward (network/layer.py:21-23) and once
    # more by UpScaler2D.forward (network/model.py:62).  With SiLU that is SiLU(SiLU(conv)), not idempotent.
    x = act(act(F.conv2d(x, p['up_scaler.conv.conv_layer.weight'], p['up_scaler.conv.conv_layer.bias'], padding=1)))
    x = F.interpolate(x, size=rs[4], mode='bilinear', align_corners=True)
    return x.permute(0, 2, 3, 1).contiguous()


def decoder_regressor(x: Tensor, grid: Tensor, p: Dict[str, Tensor], cfg: dict, taps: dict = None) -> Tensor:
    """Sp_DecoderRegressor.forward (network/sp_model.py:53-64)."""
    pre = 'decoder_regressor.'
    x = torch.cat([x, grid], dim=-1)
    x = F.linear(x, p[pre + 'spatial_fc_layer.weight'], p[pre + 'spatial_fc_layer.bias'])
    if taps is not None:
        taps['spatial_fc'] = x
    for i in range(cfg['num_decoder_layer']):
        x = spectral_conv2d(x, p, f'{pre}layers.{i}.', cfg['num_frequence_mode'], cfg['acti_decoder_layer'])
        if taps is not None:
            taps[f'spectral{i}'] = x
    return feed_forward(x, p, pre + 'ffn_layer.', cfg['acti_decoder_layer'])


def model_forward(node: Tensor, position: Tensor, grid: Tensor, p: Dict[str, Tensor], cfg: dict, taps: dict = None) -> Tensor:
    """Sp_GalerkinTransformer2D.forward (network/sp_model.py:91-113), drop rates 0.

    node [N,r,r,1], position [N,ra,ra,2], grid [N,r,r,2] -> [N,r,r,1].
    De-normalisation X*(std+1e-5)+mean follows dataset/darcy_dataset.py:30-31 with
    cfg['target_mean'], cfg['target_std'] (defaults 0 and 1: GaussNormalizer() with no data, :23-25).
    """
    x = down_scaler(node, p, cfg)
    if taps is not None:
        taps['down'] = x
    N, ra, _, D = x.shape
    x = x.view(N, ra * ra, D)
    pos = position.reshape(N, ra * ra, -1)
    for i in range(cfg['num_encoder_layer']):
        lt = {} if taps is not None else None
        x = encoder_layer(x, pos, p, f'encoder_mixer.layers.{i}.', cfg, lt)
        if taps is not None:
            taps[f'enc{i}'] = x
            if i == 0:
                taps.update({f'enc0_{k}': v for k, v in lt.items()})
    x = x.view(N, ra, ra, D)
    x = up_scaler(x, p, cfg)
    if taps is not None:
        taps['up'] = x
    x = decoder_regressor(x, grid, p, cfg, taps)
    if taps is not None:
        taps['decoder'] = x
    x = x * (cfg.get('target_std', 1.0) + 1.0e-5) + cfg.get('target_mean', 0.0)
    if cfg.get('boundary_condition', 'dirichlet') == 'dirichlet':
        x = F.pad(x[:, 1:-1, 1:-1].contiguous(), (0, 0, 1, 1, 1, 1), 'constant', 0)
    return x


def relative_l2_metric(pred: Tensor, target: Tensor, eps: float = 1.0e-10) -> Tensor:
    """mean over samples of sqrt(mean((p-t)^2) / (mean(t^2) + eps))  (engine/metric.py:47-67, 'L1' reduction)."""
    p, t = pred.squeeze(-1), target.squeeze(-1)
    loss = (p - t).pow(2).mean(dim=[1, 2]) / (t.pow(2).mean(dim=[1, 2]) + eps)
    return loss.sqrt().mean()


# ----------------------------------------------------------------------------
# parameters and synthetic inputs
# ----------------------------------------------------------------------------
def default_config(fine_resolution: int = 421, subsample_node: int = 2, subsample_attn: int = 8,
                   num_frequence_mode: int = 12, num_encoder_layer: int = 6, num_decoder_layer: int = 2) -> dict:
    """The hyper-parameters of config/darcy_config.yaml that the forward uses, with every drop rate 0."""
    r = int((fine_resolution - 1) / subsample_node + 1)
    ra = int((fine_resolution - 1) / subsample_attn + 1)
    return dict(
        fine_resolution=fine_resolution, subsample_node=subsample_node, subsample_attn=subsample_attn,
        r=r, r_attn=ra, resolution_size=get_resolution_size(r, ra),
        dim_node=1, dim_target=1, dim_position=2, boundary_condition='dirichlet',
        dim_hidden=128, num_head=4, num_encoder_layer=num_encoder_layer, attn_norm_eps=1.0e-6,
        attn_xavier=0.01, attn_diagonal=0.01, attn_symmetric=False,
        dim_encoder_ffn=256, acti_encoder_ffn='relu', acti_downscaler='relu', acti_upscaler='silu',
        num_decoder_layer=num_decoder_layer, acti_decoder_layer='silu', dim_spatial_hidden=32,
        num_frequence_mode=num_frequence_mode, target_mean=0.0, target_std=1.0,
    )


def to_dtype(p: Dict[str, Tensor], dtype) -> Dict[str, Tensor]:
    return {k: v.to(dtype) for k, v in p.items()}


def gaussian_random_field(S: int, rng: np.random.Generator, alpha: float = 2.0, tau: float = 3.0) -> np.ndarray:
    """One GRF sample on an S x S grid: L = S * tau^(alpha-1) * (pi^2 (k1^2+k2^2) + tau^2)^(-alpha/2) * N(0,1),
    L[0,0] = 0, U = idct2(L)   (dataset/darcy_generate/Gaussian_Random_Field.m:10-19)."""
    import scipy.fft
    k1, k2 = np.meshgrid(np.arange(S), np.arange(S))
    coef = tau ** (alpha - 1) * (np.pi ** 2 * (k1 ** 2 + k2 ** 2) + tau ** 2) ** (-alpha / 2)
    L = S * coef * rng.standard_normal((S, S))
    L[0, 0] = 0.0
    return scipy.fft.idctn(L, type=2, norm='ortho')


def darcy_coefficient(n: int, S: int, sub: int, seed: int) -> np.ndarray:
    """Thresholded coefficient fields a = 12 where U >= 0 else 3 (dataset/darcy_generate/Darcy_Gen.m:35-37),
    sub-sampled [::sub, ::sub]; float32 [n, r, r, 1]."""
    out = []
    for i in range(n):
        rng = np.random.default_rng([seed, i])
        U = gaussian_random_field(S, rng)
        out.append(np.where(U >= 0, 12.0, 3.0)[::sub, ::sub])
    a = np.stack(out).astype(np.float32)
    return a[..., None]
