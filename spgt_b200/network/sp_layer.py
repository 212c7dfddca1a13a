"""Sp_GalerkinAttention / Sp_EncoderLayer / Sp_SpectralConv2D: same constructors, parameter names and forward
signatures as the reference's network/sp_layer.py.  `forward` is the inference path, every step on the sm_100a kernels;
`forward_train` is the differentiable path the training loop uses (the reference's own op sequence: this library's
attention / projection / data-movement ops with their backward kernels, library ops for the rest).

Dropout: the reference calls F.dropout without `training=`, which keeps it active under model.eval()
(network/sp_layer.py:76,133).  These modules treat every drop rate as 0; use rates of 0 in the reference when
comparing outputs.
"""
import math

import torch
from torch import Tensor

from .. import ops
from .layer import FeedForward, _KernelWeights, _act, _linear_kn, _linear_tc


class Sp_GalerkinAttention(_KernelWeights):
    def __init__(self, dim_hidden, num_head, dim_position, norm_eps, attn_droprate, fc_droprate, xavier, diagonal,
                 symmetric) -> None:
        super().__init__()
        assert dim_hidden % 128 == 0 and dim_hidden // num_head == 32
        dim_head = dim_hidden // num_head
        self.dim_hidden, self.num_head, self.dim_head, self.dim_position = dim_hidden, num_head, dim_head, dim_position
        self.norm_eps, self.attn_droprate, self.fc_droprate = norm_eps, attn_droprate, fc_droprate
        P, E = torch.nn.Parameter, torch.empty
        self.weight_Q, self.weight_K, self.weight_V = (P(E([dim_hidden, dim_hidden])) for _ in range(3))
        self.bias_Q, self.bias_K, self.bias_V = (P(E([dim_hidden])) for _ in range(3))
        self.ln_weight_K, self.ln_weight_V = (P(E([num_head, dim_head])) for _ in range(2))
        self.ln_bias_K, self.ln_bias_V = (P(E([num_head, dim_head])) for _ in range(2))
        self.fc_layer = torch.nn.Linear(dim_hidden + dim_position * num_head, dim_hidden)
        self._reset_parameters(xavier, diagonal, symmetric)

    def _reset_parameters(self, xavier, diagonal, symmetric):
        # same initialisation as the reference (network/sp_layer.py:39-50)
        for weight in [self.weight_Q, self.weight_K, self.weight_V]:
            torch.nn.init.xavier_uniform_(weight, gain=xavier)
            if diagonal > 0:
                weight.data += diagonal * torch.diag(torch.ones(weight.size(-1)))
            if symmetric:
                weight.data += weight.data.T
        for bias in [self.bias_Q, self.bias_K, self.bias_V]:
            torch.nn.init.constant_(bias, 0)
        for lnw, lnb in zip([self.ln_weight_K, self.ln_weight_V], [self.ln_bias_K, self.ln_bias_V]):
            torch.nn.init.ones_(lnw)
            torch.nn.init.zeros_(lnb)

    def forward(self, Q: Tensor, K: Tensor, V: Tensor, position: Tensor, residual: Tensor = None) -> Tensor:
        """Q,K,V [N,S,D], position [N,S,d_pos] -> [N,S,D] (+ residual, fused into the output projection).
        When Q, K and V are the same tensor (self-attention) all three projections run in one launch."""
        d = lambda t: t.detach()
        H, dh, dp = self.num_head, self.dim_head, self.dim_position
        if Q is K and K is V and self.dim_hidden == 128:
            wqkv = self._cached('wqkv', lambda: ops.TcWeight(
                torch.cat([d(self.weight_Q), d(self.weight_K), d(self.weight_V)], dim=1).contiguous()))
            q, k, v = ops.projpos_qkv_tc(
                Q, wqkv, d(self.bias_Q), d(self.bias_K), d(self.bias_V), d(self.ln_weight_K), d(self.ln_bias_K),
                d(self.ln_weight_V), d(self.ln_bias_V), self.norm_eps, position, H, dh, dp)
        elif Q is K and K is V:
            q, k, v = ops.projpos_qkv(
                Q, d(self.weight_Q), d(self.bias_Q), d(self.weight_K), d(self.bias_K), d(self.weight_V), d(self.bias_V),
                d(self.ln_weight_K), d(self.ln_bias_K), d(self.ln_weight_V), d(self.ln_bias_V), self.norm_eps, position,
                H, dh, dp)
        else:
            q = ops.projpos(Q, d(self.weight_Q), d(self.bias_Q), position, H, dh, dp)
            k = ops.projpos_lnorm(K, d(self.weight_K), d(self.bias_K), d(self.ln_weight_K), d(self.ln_bias_K), position,
                                  self.norm_eps, H, dh, dp)
            v = ops.projpos_lnorm(V, d(self.weight_V), d(self.bias_V), d(self.ln_weight_V), d(self.ln_bias_V), position,
                                  self.norm_eps, H, dh, dp)
        X = ops.galerkin_attention(q, k, v, merged_heads=True)          # [N, S, H*(d_pos+d_head)]
        wfc = self._cached('fc', lambda: _linear_tc(self.fc_layer.weight))
        return ops.linear_tc(X, wfc, d(self.fc_layer.bias), None, residual)


def _attention_forward_train(self, Q: Tensor, K: Tensor, V: Tensor, position: Tensor) -> Tensor:
    """Sp_GalerkinAttention.forward of the reference (network/sp_layer.py:52-78, drop rates 0) on the differentiable ops."""
    from ..extension.bind.galerkin_attention import (multihead_galerkin_attention_cccr_cuda,
                                                     multihead_projection_layernorm_with_position_rrc_cuda,
                                                     multihead_projection_with_position_rrc_cuda)
    H, dh, dp = self.num_head, self.dim_head, self.dim_position
    N, S, _ = Q.shape
    q = multihead_projection_with_position_rrc_cuda(Q, self.weight_Q, self.bias_Q, position, H, dh, dp)
    k = multihead_projection_layernorm_with_position_rrc_cuda(K, self.weight_K, self.bias_K, self.ln_weight_K, self.ln_bias_K,
                                                             position, self.norm_eps, H, dh, dp)
    v = multihead_projection_layernorm_with_position_rrc_cuda(V, self.weight_V, self.bias_V, self.ln_weight_V, self.ln_bias_V,
                                                             position, self.norm_eps, H, dh, dp)
    X = multihead_galerkin_attention_cccr_cuda(q, k, v)                  # [N, H, S, d_pos + d_head]
    X = X.transpose(1, 2).contiguous().view(N, S, H * (dp + dh))
    return self.fc_layer(X)


Sp_GalerkinAttention.forward_train = _attention_forward_train


class Sp_EncoderLayer(torch.nn.Module):
    def __init__(self, dim_hidden, num_head, dim_position, norm_eps, attn_droprate, fc_droprate, xavier, diagonal,
                 symmetric, ffn_dim_hidden, ffn_droprate, ffn_activation) -> None:
        super().__init__()
        self.attention_layer = Sp_GalerkinAttention(
            dim_hidden, num_head, dim_position, norm_eps, attn_droprate, fc_droprate, xavier, diagonal, symmetric)
        self.ffn_layer = FeedForward(dim_hidden, dim_hidden, ffn_dim_hidden, ffn_droprate, ffn_activation)

    def forward(self, X: Tensor, position: Tensor) -> Tensor:
        """X [N,S,D], position [N,S,d_pos] -> X + attention(X) then + ffn(.)  (network/sp_layer.py:94-104)."""
        X = self.attention_layer(X, X, X, position, residual=X)
        return self.ffn_layer(X, residual=X)

    def forward_train(self, X: Tensor, position: Tensor) -> Tensor:
        X = X + self.attention_layer.forward_train(X, X, X, position)
        return X + self.ffn_layer.forward_train(X)


class Sp_SpectralConv2D(_KernelWeights):
    """structure='fused' (default): one mode-truncated DFT pipeline (spgt_spectral_conv2d_fwd).
    structure='reference': the reference's own op sequence (network/sp_layer.py:125-156): batched_transpose ->
    torch.fft.rfft2 -> transpose_gather_dual -> complex matmul -> transpose_scatter_dual -> torch.fft.irfft2 ->
    batched_transpose, which exercises the data-movement ops in context."""

    def __init__(self, in_dim, out_dim, mode, droprate, activation, structure: str = 'fused') -> None:
        super().__init__()
        self.in_dim, self.out_dim, self.mode, self.droprate = in_dim, out_dim, mode, droprate
        self.activation = activation
        self.structure = structure
        self.residual_layer = torch.nn.Linear(in_dim, out_dim)
        self.fourier_weight = torch.nn.ParameterList([
            torch.nn.Parameter(torch.empty([mode, mode, in_dim, out_dim, 2])) for _ in range(2)])
        for param in self.fourier_weight:
            torch.nn.init.xavier_normal_(param, gain=1.0 / (in_dim * out_dim) * math.sqrt(in_dim + out_dim))

    def forward(self, X: Tensor) -> Tensor:
        N, r, _, in_dim = X.shape
        m, out_dim = self.mode, self.out_dim
        wr = self._cached('wr', lambda: _linear_kn(self.residual_layer.weight))
        br = self.residual_layer.bias.detach()
        fw0, fw1 = self.fourier_weight[0].detach(), self.fourier_weight[1].detach()
        if self.structure == 'fused':
            return ops.spectral_conv2d(X, wr, br, fw0, fw1, m, self.activation)
        from ..extension.bind.datamove import batched_transpose, transpose_gather_dual, transpose_scatter_dual
        Xt = batched_transpose(X, [N], [r, r], [in_dim])
        X_ft = torch.fft.rfft2(Xt, s=(r, r), norm='ortho').contiguous()
        a, b = transpose_gather_dual(X_ft, [N, in_dim], r, r // 2 + 1, m, m, 0, 0, r - m, 0)
        a = a @ torch.view_as_complex(fw0)
        b = b @ torch.view_as_complex(fw1)
        Out_ft = transpose_scatter_dual(a.contiguous(), b.contiguous(), [N, out_dim], r, r // 2 + 1, m, m, 0, 0, r - m, 0)
        Y = torch.fft.irfft2(Out_ft, s=(r, r), norm='ortho').contiguous()
        Y = batched_transpose(Y, [N], [out_dim], [r, r])
        res = ops.linear(X, wr, br, out_dim, None, Y)             # X @ Wr + br + Y
        return torch.nn.functional.silu(res) if self.activation == 'silu' else torch.relu(res)

    def forward_train(self, X: Tensor) -> Tensor:
        """Differentiable path: the reference's op sequence (network/sp_layer.py:125-156, drop rate 0)."""
        from ..extension.bind.datamove import batched_transpose, transpose_gather_dual, transpose_scatter_dual
        N, r, _, in_dim = X.shape
        m, out_dim = self.mode, self.out_dim
        res = self.residual_layer(X)
        Xt = batched_transpose(X.contiguous(), [N], [r, r], [in_dim])
        X_ft = torch.fft.rfft2(Xt, s=(r, r), norm='ortho').contiguous()
        a, b = transpose_gather_dual(X_ft, [N, in_dim], r, r // 2 + 1, m, m, 0, 0, r - m, 0)
        a = a @ torch.view_as_complex(self.fourier_weight[0])
        b = b @ torch.view_as_complex(self.fourier_weight[1])
        Out_ft = transpose_scatter_dual(a.contiguous(), b.contiguous(), [N, out_dim], r, r // 2 + 1, m, m, 0, 0, r - m, 0)
        Y = torch.fft.irfft2(Out_ft, s=(r, r), norm='ortho').contiguous()
        Y = batched_transpose(Y, [N], [out_dim], [r, r])
        return _act(self.activation)(Y + res)
