"""Drop-in for the reference's extension/bind/datamove.py: same names and signatures as extension/bind/datamove.py:68-87,
differentiable like the reference's autograd functions (:13-65) - the backward of each data-movement op is another
data-movement op of this library."""
import torch
from torch import Tensor

from ... import ops


def _needs_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


class Batched_Transpose_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, batch_list, M_list, N_list):
        ctx.lists = (list(batch_list), list(M_list), list(N_list))
        return ops.batched_transpose(X.contiguous(), batch_list, M_list, N_list)

    @staticmethod
    def backward(ctx, grad_out):
        batch_list, M_list, N_list = ctx.lists
        return ops.batched_transpose(grad_out.contiguous(), batch_list, N_list, M_list), None, None, None


class Transpose_Gather_Dual_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, dim_list, *geom):
        ctx.extras = (list(dim_list), geom)
        return ops.transpose_gather_dual(src.contiguous(), dim_list, *geom)

    @staticmethod
    def backward(ctx, grad_out1, grad_out2):
        dim_list, geom = ctx.extras
        grad_src = ops.transpose_scatter_dual(grad_out1.contiguous(), grad_out2.contiguous(), dim_list, *geom)
        return (grad_src, None) + (None,) * len(geom)


class Transpose_Scatter_Dual_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src1, src2, dim_list, *geom):
        ctx.extras = (list(dim_list), geom)
        return ops.transpose_scatter_dual(src1.contiguous(), src2.contiguous(), dim_list, *geom)

    @staticmethod
    def backward(ctx, grad_out):
        dim_list, geom = ctx.extras
        g1, g2 = ops.transpose_gather_dual(grad_out.contiguous(), dim_list, *geom)
        return (g1, g2, None) + (None,) * len(geom)


def batched_transpose(X: Tensor, batch_list: list, M_list: list, N_list: list) -> Tensor:
    """[batch..., M..., N...] -> [batch..., N..., M...]."""
    if _needs_grad(X):
        return Batched_Transpose_Function.apply(X, batch_list, M_list, N_list)
    return ops.batched_transpose(X, batch_list, M_list, N_list)


def transpose_gather_dual(src: Tensor, dim_list: list, H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2):
    """complex64 [dim..., H_all, W_all] -> two [H_low, W_low, dim...] blocks."""
    geom = (H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2)
    if _needs_grad(src):
        return Transpose_Gather_Dual_Function.apply(src, dim_list, *geom)
    return ops.transpose_gather_dual(src, dim_list, *geom)


def transpose_scatter_dual(src1: Tensor, src2: Tensor, dim_list: list, H_all, W_all, H_low, W_low,
                           H_base_1, W_base_1, H_base_2, W_base_2) -> Tensor:
    """Inverse of transpose_gather_dual; everything outside the two blocks is zero."""
    geom = (H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2)
    if _needs_grad(src1, src2):
        return Transpose_Scatter_Dual_Function.apply(src1, src2, dim_list, *geom)
    return ops.transpose_scatter_dual(src1, src2, dim_list, *geom)
