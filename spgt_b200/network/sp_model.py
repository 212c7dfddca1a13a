"""Sp_EncoderMixer / Sp_DecoderRegressor / Sp_GalerkinTransformer2D: same constructors, parameter names
(state_dict keys) and forward signatures as the reference's network/sp_model.py.  Without gradients (eval, or
torch.no_grad) the forward runs on the fused inference kernels; in training mode with gradients enabled it runs the
differentiable path (`forward_train` of the modules)."""
import numpy as np
import torch
from torch import Tensor

from .. import ops
from .layer import FeedForward, _KernelWeights, _linear_kn, _linear_tc
from .model import DownScaler2D, UpScaler2D
from .sp_layer import Sp_EncoderLayer, Sp_SpectralConv2D


class Sp_EncoderMixer(torch.nn.Module):
    def __init__(self, num_layer, dim_hidden, num_head, dim_position, norm_eps, attn_droprate, fc_droprate, xavier,
                 diagonal, symmetric, ffn_dim_hidden, ffn_droprate, ffn_activation) -> None:
        super().__init__()
        self.layers = torch.nn.ModuleList([
            Sp_EncoderLayer(dim_hidden, num_head, dim_position, norm_eps, attn_droprate, fc_droprate, xavier, diagonal,
                            symmetric, ffn_dim_hidden, ffn_droprate, ffn_activation) for _ in range(num_layer)])

    def forward(self, X: Tensor, position: Tensor) -> Tensor:
        N, r_attn, _, dim_hidden = X.shape
        X = X.view(N, r_attn * r_attn, dim_hidden)
        position = position.reshape(N, r_attn * r_attn, position.size(-1))
        for layer in self.layers:
            X = layer(X, position)
        return X.view(N, r_attn, r_attn, dim_hidden)

    def forward_train(self, X: Tensor, position: Tensor) -> Tensor:
        N, r_attn, _, dim_hidden = X.shape
        X = X.reshape(N, r_attn * r_attn, dim_hidden)
        position = position.reshape(N, r_attn * r_attn, position.size(-1)).contiguous()
        for layer in self.layers:
            X = layer.forward_train(X, position)
        return X.view(N, r_attn, r_attn, dim_hidden)


class Sp_DecoderRegressor(_KernelWeights):
    def __init__(self, num_layer, in_dim, out_dim, dim_position, dim_spatial_hidden, mode, droprate, activation) -> None:
        super().__init__()
        assert out_dim == 1, 'the fused decoder head produces the scalar Darcy target'
        self.in_dim, self.dim_position, self.activation = in_dim, dim_position, activation
        self.spatial_fc_layer = torch.nn.Linear(in_dim + dim_position, dim_spatial_hidden)
        self.layers = torch.nn.ModuleList([
            Sp_SpectralConv2D(dim_spatial_hidden, dim_spatial_hidden, mode, droprate, activation) for _ in range(num_layer)])
        dim_ffn_hidden = 2 * dim_position * dim_spatial_hidden
        self.ffn_layer = FeedForward(dim_spatial_hidden, out_dim, dim_ffn_hidden, droprate, activation)

    def _spectral_and_head(self, X: Tensor, scale, shift, dirichlet, scale_map=None, shift_map=None) -> Tensor:
        for layer in self.layers:
            X = layer(X)
        f = self.ffn_layer
        w2 = self._cached('w2', lambda: f.layer2.weight.detach().reshape(-1).contiguous())
        b2 = self._cached('b2', lambda: float(f.layer2.bias.detach().reshape(-1)[0]))
        if f.layer1.out_features == 128:
            w1 = self._cached('w1tc', lambda: _linear_tc(f.layer1.weight))
            return ops.decoder_head_tc(X, w1, f.layer1.bias.detach(), w2, b2, scale, shift, dirichlet, self.activation,
                                       scale_map, shift_map)
        w1 = self._cached('w1', lambda: _linear_kn(f.layer1.weight))
        return ops.decoder_head(X, w1, f.layer1.bias.detach(), w2, b2, scale, shift, dirichlet, self.activation,
                                scale_map, shift_map)

    def forward(self, X: Tensor, grid: Tensor = None) -> Tensor:
        """X [N,r,r,in_dim], grid [N,r,r,d_pos] -> [N,r,r,1]  (network/sp_model.py:53-64)."""
        return self._spectral_and_head(self._fc_split(X, grid), 1.0, 0.0, False)

    def forward_train(self, X: Tensor, grid: Tensor) -> Tensor:
        """Differentiable path (network/sp_model.py:53-64)."""
        X = self.spatial_fc_layer(torch.concat([X, grid], dim=-1))
        for layer in self.layers:
            X = layer.forward_train(X)
        return self.ffn_layer.forward_train(X)

    def _fc_split(self, X, grid):
        """spatial_fc_layer(concat(X, grid)) = X @ Wx + grid @ Wg + b without materialising the concatenation."""
        wx, wg = self._split_fc()
        uw = ops.linear_tc(X, wx, None, None)
        return ops.upsample_grid(uw, grid, wg, self.spatial_fc_layer.bias.detach(), X.shape[1], X.shape[2])

    def _split_fc(self):
        w = self.spatial_fc_layer.weight
        wx = self._cached('wx', lambda: _linear_tc(w[:, :self.in_dim]))
        wg = self._cached('wg', lambda: w.detach()[:, self.in_dim:].t().contiguous())
        return wx, wg

    def forward_from_mid(self, U: Tensor, grid: Tensor, scale, shift, dirichlet, scale_map=None, shift_map=None) -> Tensor:
        """U [N,r_mid,r_mid,in_dim] is the up-scaler output BEFORE its last interpolation.  Interpolation and
        Linear are both linear maps, so Linear(concat(resize(U), grid)) = resize(U @ Wx) + grid @ Wg + b: the
        in_dim-channel full-resolution tensor is never formed."""
        wx, wg = self._split_fc()
        uw = ops.linear_tc(U, wx, None, None)
        X = ops.upsample_grid(uw, grid, wg, self.spatial_fc_layer.bias.detach(), grid.shape[1], grid.shape[2])
        return self._spectral_and_head(X, scale, shift, dirichlet, scale_map, shift_map)


def _normalizer_affine(normalizer, r: int, device):
    """(scale, shift, scale_map, shift_map) of inverse_transform(X) = X * (std + eps) + mean."""
    if normalizer is None:
        return 1.0, 0.0, None, None
    eps = float(getattr(normalizer, 'eps', 1.0e-5))
    mean = torch.as_tensor(np.asarray(normalizer.mean.cpu() if isinstance(normalizer.mean, torch.Tensor) else normalizer.mean),
                           dtype=torch.float32)
    std = torch.as_tensor(np.asarray(normalizer.std.cpu() if isinstance(normalizer.std, torch.Tensor) else normalizer.std),
                          dtype=torch.float32)
    if mean.numel() == 1 and std.numel() == 1:
        return float(std.reshape(-1)[0]) + eps, float(mean.reshape(-1)[0]), None, None
    scale_map = (std.reshape(-1) + eps).expand(r * r).contiguous().to(device) if std.numel() in (1, r * r) else None
    shift_map = mean.reshape(-1).expand(r * r).contiguous().to(device) if mean.numel() in (1, r * r) else None
    if scale_map is None or shift_map is None:
        raise ValueError('target normalizer statistics must be scalars or one value per grid node')
    return 1.0, 0.0, scale_map, shift_map


class Sp_GalerkinTransformer2D(torch.nn.Module):
    """Darcy Galerkin Transformer forward: down-scaler -> encoder layers -> up-scaler -> spectral regressor ->
    de-normalisation -> Dirichlet frame (network/sp_model.py:67-113).  cfg carries the keys of the reference's
    config (config/darcy_config.yaml) plus 'resolution_size' and 'target_normalizer'."""

    def __init__(self, cfg) -> None:
        super().__init__()
        self.droprate = cfg['drop_module']
        self.boundary_condition = cfg['boundary_condition']
        self.normalizer = cfg.get('target_normalizer')
        self.down_scaler = DownScaler2D(cfg['resolution_size'], cfg['dim_node'], cfg['dim_hidden'], cfg['drop_downscaler'],
                                        cfg['acti_downscaler'])
        self.encoder_mixer = Sp_EncoderMixer(
            cfg['num_encoder_layer'], cfg['dim_hidden'], cfg['num_head'], cfg['dim_position'], cfg['attn_norm_eps'],
            cfg['drop_encoder_attn'], cfg['drop_encoder_attn_fc'], cfg['attn_xavier'], cfg['attn_diagonal'],
            cfg['attn_symmetric'], cfg['dim_encoder_ffn'], cfg['drop_encoder_ffn'], cfg['acti_encoder_ffn'])
        self.up_scaler = UpScaler2D(cfg['resolution_size'], cfg['dim_hidden'], cfg['dim_hidden'], cfg['drop_upscaler'],
                                    cfg['acti_upscaler'])
        self.decoder_regressor = Sp_DecoderRegressor(
            cfg['num_decoder_layer'], cfg['dim_hidden'], cfg['dim_target'], cfg['dim_position'], cfg['dim_spatial_hidden'],
            cfg['num_frequence_mode'], cfg['drop_decoder_layer'], cfg['acti_decoder_layer'])
        self._affine = None

    def forward(self, X: Tensor, position: Tensor, grid: Tensor, taps: dict = None) -> Tensor:
        """X [N,r,r,1], position [N,r_attn,r_attn,2], grid [N,r,r,2] -> [N,r,r,1]; CUDA fp32 contiguous tensors.
        `taps`, when a dict, receives intermediate tensors (down-scaler output, each encoder layer, ...).
        In training mode with gradients enabled the differentiable path runs; otherwise the fused inference kernels."""
        if self.training and torch.is_grad_enabled():
            return self.forward_train(X, position, grid)
        with torch.no_grad():
            return self._forward_fused(X, position, grid, taps)

    def forward_train(self, X: Tensor, position: Tensor, grid: Tensor) -> Tensor:
        """The reference's forward (network/sp_model.py:91-113, every drop rate 0) on differentiable ops."""
        X = self.down_scaler.forward_train(X)
        X = self.encoder_mixer.forward_train(X, position)
        X = self.up_scaler.forward_train(X)
        X = self.decoder_regressor.forward_train(X, grid)
        r = X.shape[1]
        scale, shift, scale_map, shift_map = _normalizer_affine(self.normalizer, r, X.device)    # X * (std + eps) + mean
        X = X * (scale if scale_map is None else scale_map.view(1, r, r, 1)) + (shift if shift_map is None else shift_map.view(1, r, r, 1))
        if self.boundary_condition == 'dirichlet':
            X = torch.nn.functional.pad(X[:, 1:-1, 1:-1].contiguous(), (0, 0, 1, 1, 1, 1), 'constant', 0)
        return X

    def _forward_fused(self, X: Tensor, position: Tensor, grid: Tensor, taps: dict = None) -> Tensor:
        r = X.shape[1]
        if self._affine is None or self._affine[0] != (r, X.device):
            self._affine = ((r, X.device), _normalizer_affine(self.normalizer, r, X.device))
        scale, shift, scale_map, shift_map = self._affine[1]
        X = self.down_scaler(X)
        if taps is not None:
            taps['down'] = X
        N, ra, _, D = X.shape
        pos = position.reshape(N, ra * ra, position.size(-1))
        X = X.view(N, ra * ra, D)
        for i, layer in enumerate(self.encoder_mixer.layers):
            X = layer(X, pos)
            if taps is not None:
                taps[f'enc{i}'] = X
        U = self.up_scaler.forward_mid(X.view(N, ra, ra, D))
        if taps is not None:
            taps['up_mid'] = U
        return self.decoder_regressor.forward_from_mid(U, grid, scale, shift, self.boundary_condition == 'dirichlet',
                                                       scale_map, shift_map)
