"""Shared layers of the Darcy model with the reference's parameter names (network/layer.py).

Each module keeps ordinary torch Parameters (so a reference state_dict loads unchanged) and a cache of the same
weights re-laid-out for the kernels ([K, N] row-major, column count padded to a multiple of 4).  `forward` is the
inference path on the fused kernels; `forward_train` is the differentiable path of the training loop, which - like
the reference's own SpGT training - runs the convolutions, interpolations, dense layers and FFTs as library ops
under torch autograd and the attention / projection / data-movement steps on this library's ops and their backward
kernels.
"""
import torch
from torch import Tensor

from .. import ops


class _KernelWeights(torch.nn.Module):
    """Caches derived weight layouts; the cache is dropped whenever parameters are (re)loaded or moved."""

    def __init__(self):
        super().__init__()
        self._kw = {}
        self.register_load_state_dict_post_hook(lambda module, incompatible: module._kw.clear())

    def _apply(self, fn, *args, **kwargs):
        self._kw.clear()
        return super()._apply(fn, *args, **kwargs)

    def _cached(self, key, make):
        """Derived layout of the module's weights, rebuilt when a parameter has been modified in place since it was
        made (an optimizer step bumps the parameters' version counters)."""
        tag = sum(p._version for p in self.parameters())
        hit = self._kw.get(key)
        if hit is None or hit[0] != tag:
            with torch.no_grad():
                hit = (tag, make())
            self._kw[key] = hit
        return hit[1]


def _linear_kn(weight: Tensor) -> Tensor:
    """torch Linear weight [out, in] -> [in, out4] row-major."""
    return ops.pad_cols(weight.detach().t().contiguous())


def _conv_kn(weight: Tensor) -> Tensor:
    """Conv2d weight [Cout, Cin, 3, 3] -> [(ky*3+kx)*Cin + ci, Cout4] row-major."""
    cout, cin = weight.shape[:2]
    return ops.pad_cols(weight.detach().permute(2, 3, 1, 0).reshape(9 * cin, cout).contiguous())


def _linear_tc(weight: Tensor) -> 'ops.TcWeight':
    """torch Linear weight [out, in] prepared for the tcgen05 GEMM."""
    return ops.TcWeight(weight.detach().t().contiguous())


def _conv_tc(weight: Tensor, bias: Tensor, cin_pad: int, cout_pad: int):
    """Conv2d weight [Cout, Cin, 3, 3] (+ bias) prepared for the tcgen05 implicit GEMM, with input / output channels
    zero-padded to cin_pad / cout_pad (padded outputs come out as act(0))."""
    cout, cin = weight.shape[:2]
    w = torch.zeros(cout_pad, cin_pad, 3, 3, device=weight.device, dtype=weight.dtype)
    w[:cout, :cin] = weight.detach()
    b = torch.zeros(cout_pad, device=weight.device, dtype=weight.dtype)
    b[:cout] = bias.detach()
    return ops.TcWeight(w.permute(2, 3, 1, 0).reshape(9 * cin_pad, cout_pad).contiguous()), b


class ConvResBlock2D(_KernelWeights):
    """conv3x3(pad 1) -> [dropout, rate treated as 0] -> activation; NHWC in and out.
    Reference: network/layer.py:7-24 (NCHW there; the kernels keep channels last throughout)."""

    def __init__(self, in_dim, out_dim, kernel_size, padding, droprate, activation) -> None:
        super().__init__()
        assert kernel_size == 3 and padding == 1
        self.droprate = droprate
        self.activation = activation
        self.conv_layer = torch.nn.Conv2d(in_dim, out_dim, kernel_size=kernel_size, padding=padding)

    def kernel_weight(self):
        return self._cached('w', lambda: _conv_kn(self.conv_layer.weight))

    def forward_train(self, X: Tensor) -> Tensor:
        """NCHW in and out, differentiable (network/layer.py:16-24 with drop rate 0)."""
        return _act(self.activation)(self.conv_layer(X))

    def forward_nhwc(self, X: Tensor, cin_off: int, out: Tensor, cout_off: int, act=None) -> Tensor:
        """Generic path (any even channel counts / offsets): warp-MMA implicit GEMM."""
        w = self.conv_layer.weight
        return ops.conv3x3(X, cin_off, w.shape[1], self.kernel_weight(), self.conv_layer.bias.detach(), out, cout_off,
                           w.shape[0], self.activation if act is None else act)

    def forward_tc(self, X: Tensor, cin_pad: int, cout_pad: int, act=None) -> Tensor:
        """tcgen05 path: X [N,H,W,cin_pad] (channels beyond in_dim must be finite; their weights are zero) ->
        new tensor [N,H,W,cout_pad] whose channels beyond out_dim hold act(0)."""
        wt, b = self._cached(('tc', cin_pad, cout_pad),
                             lambda: _conv_tc(self.conv_layer.weight, self.conv_layer.bias, cin_pad, cout_pad))
        out = torch.empty(*X.shape[:3], cout_pad, device=X.device, dtype=X.dtype)
        return ops.conv3x3_tc(X, 0, cin_pad, wt, b, out, 0, cout_pad, self.activation if act is None else act)


def _act(name):
    """The reference selects SiLU for 'silu' and ReLU for any other string (network/layer.py:14,163)."""
    return torch.nn.functional.silu if name == 'silu' else torch.relu


class FeedForward(_KernelWeights):
    """Linear -> activation -> Linear (dropout rate treated as 0).  Reference: network/layer.py:155-174."""

    def __init__(self, in_dim, out_dim, dim_hidden, droprate, activation) -> None:
        super().__init__()
        self.droprate = droprate
        self.activation = activation
        self.layer1 = torch.nn.Linear(in_dim, dim_hidden)
        self.layer2 = torch.nn.Linear(dim_hidden, out_dim)
        self.fused = True        # one kernel for both GEMMs when the shape is 128 -> 256 -> 128

    def forward(self, X: Tensor, residual: Tensor = None) -> Tensor:
        """X [..., in_dim] -> [..., out_dim] (+ residual when given, fused into the second GEMM)."""
        w1 = self._cached('w1', lambda: _linear_tc(self.layer1.weight))
        w2 = self._cached('w2', lambda: _linear_tc(self.layer2.weight))
        if self.fused and w1.K == 128 and w1.N == 256 and w2.N == 128:
            return ops.ffn_tc(X, w1, self.layer1.bias.detach(), w2, self.layer2.bias.detach(), self.activation, residual)
        h = ops.linear_tc(X, w1, self.layer1.bias.detach(), self.activation)
        return ops.linear_tc(h, w2, self.layer2.bias.detach(), None, residual)

    def forward_train(self, X: Tensor) -> Tensor:
        return self.layer2(_act(self.activation)(self.layer1(X)))
