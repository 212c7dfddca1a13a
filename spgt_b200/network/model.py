"""DownScaler2D / UpScaler2D with the reference's parameter names (network/model.py:7-65)."""
import torch
from torch import Tensor
from torch.nn.functional import interpolate

from .. import ops
from .layer import ConvResBlock2D, _KernelWeights, _act


class DownScaler2D(_KernelWeights):
    """[N,r,r,1] -> [N,r_attn,r_attn,out_dim]:
    conv0+act -> bilinear to r_mid -> act -> conv1, conv2, conv3 (+act) concatenated -> bilinear to r_attn -> act.
    conv0, its activation, the first interpolation and the activation after it run as one kernel, so the
    out_dim-channel full-resolution tensor is never written; conv1..3 write straight into their channel slice
    of the concatenated tensor."""

    def __init__(self, resolution_size, in_dim, out_dim, droprate, activation) -> None:
        super().__init__()
        assert in_dim == 1, 'the fused first stage handles the single-channel Darcy coefficient'
        self.resolution_size = resolution_size
        self.activation = activation
        out_dim1 = out_dim // 3
        out_dim2 = out_dim // 3
        out_dim3 = int(out_dim - out_dim1 - out_dim2)
        self.dims = (out_dim1, out_dim2, out_dim3)
        self.conv0 = ConvResBlock2D(in_dim, out_dim, 3, 1, droprate, activation)
        self.conv1 = ConvResBlock2D(out_dim, out_dim1, 3, 1, droprate, activation)
        self.conv2 = ConvResBlock2D(out_dim1, out_dim2, 3, 1, droprate, activation)
        self.conv3 = ConvResBlock2D(out_dim2, out_dim3, 3, 1, droprate, activation)

    def forward(self, X: Tensor) -> Tensor:
        N, r, _, _ = X.shape
        mid, ra = self.resolution_size[1], self.resolution_size[2]
        w0 = self._cached('w0', lambda: self.conv0.conv_layer.weight.detach().reshape(-1, 9).t().contiguous())
        X = ops.conv0_down(X.reshape(N, r, r), w0, self.conv0.conv_layer.bias.detach(), mid[0], mid[1], self.activation)
        d1, d2, d3 = self.dims
        pad4 = lambda c: (c + 3) // 4 * 4          # the tcgen05 implicit GEMM wants channel counts that are multiples of 4
        X1 = self.conv1.forward_tc(X, X.shape[3], pad4(d1))
        X2 = self.conv2.forward_tc(X1, pad4(d1), pad4(d2))
        X3 = self.conv3.forward_tc(X2, pad4(d2), pad4(d3))
        return ops.bilinear_concat3(X1, X2, X3, d1, d2, d3, ra[0], ra[1], self.activation)

    def forward_train(self, X: Tensor) -> Tensor:
        """Differentiable path, the reference's op sequence (network/model.py:23-39, drop rate 0)."""
        act = _act(self.activation)
        X = X.permute(0, 3, 1, 2)
        X = self.conv0.forward_train(X)
        X = act(interpolate(X, size=self.resolution_size[1], mode='bilinear', align_corners=True))
        X1 = self.conv1.forward_train(X)
        X2 = self.conv2.forward_train(X1)
        X3 = self.conv3.forward_train(X2)
        X = torch.concat([X1, X2, X3], dim=1)
        X = act(interpolate(X, size=self.resolution_size[2], mode='bilinear', align_corners=True))
        return X.permute(0, 2, 3, 1).contiguous()


class UpScaler2D(_KernelWeights):
    """[N,r_attn,r_attn,in_dim] -> [N,r,r,out_dim]: bilinear to r_mid -> conv+act -> act -> bilinear to r.
    The activation is applied twice, as in the reference (once inside ConvResBlock2D.forward, network/layer.py:23,
    once more in UpScaler2D.forward, network/model.py:62)."""

    def __init__(self, resolution_size, in_dim, out_dim, droprate, activation) -> None:
        super().__init__()
        self.resolution_size = resolution_size
        self.droprate = droprate
        self.activation = activation
        self.conv = ConvResBlock2D(in_dim, out_dim, 3, 1, droprate, activation)

    def forward_mid(self, X: Tensor) -> Tensor:
        """Everything up to (not including) the last interpolation: [N, r_mid, r_mid, out_dim]."""
        mid = self.resolution_size[3]
        X = ops.bilinear(X, mid[0], mid[1], None)
        twice = 'silu2' if self.activation == 'silu' else 'relu'
        cin, cout = self.conv.conv_layer.in_channels, self.conv.conv_layer.out_channels
        if cin % 4 == 0 and cout % 4 == 0:
            return self.conv.forward_tc(X, cin, cout, act=twice)
        out = torch.empty(X.shape[0], mid[0], mid[1], cout, device=X.device, dtype=X.dtype)
        return self.conv.forward_nhwc(X, 0, out, 0, act=twice)

    def forward(self, X: Tensor) -> Tensor:
        r = self.resolution_size[4]
        return ops.bilinear(self.forward_mid(X), r[0], r[1], None)

    def forward_train(self, X: Tensor) -> Tensor:
        """Differentiable path (network/model.py:53-65): the activation is applied inside the block and once more."""
        X = X.permute(0, 3, 1, 2)
        X = interpolate(X, size=self.resolution_size[3], mode='bilinear', align_corners=True)
        X = _act(self.activation)(self.conv.forward_train(X))
        X = interpolate(X, size=self.resolution_size[4], mode='bilinear', align_corners=True)
        return X.permute(0, 2, 3, 1).contiguous()
