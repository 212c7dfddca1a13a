"""Drop-in for the reference's extension/bind/galerkin_attention.py (forward of every op; backward of the attention op).

Same function names, argument order and tensor layouts as the reference's public functions
(extension/bind/galerkin_attention.py:87-107); the work is done by the sm_100a kernels of libspgt_b200.so
instead of a JIT-built pybind module.  Inputs must be contiguous fp32 CUDA tensors: the reference reads raw
data pointers without checking, here a wrong device, dtype or layout raises.
"""
import torch
from torch import Tensor

from ... import ops


def _needs_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


class Multihead_Porjection_with_Position_Function(torch.autograd.Function):
    """Autograd wrapper with the reference's class name (extension/bind/galerkin_attention.py:12-34)."""

    @staticmethod
    def forward(ctx, input, weight, bias, position, num_head, dim_head, dim_position):
        input, weight = input.contiguous(), weight.contiguous()
        ctx.save_for_backward(input, weight, bias)
        ctx.dims = (num_head, dim_head, dim_position)
        return ops.projpos(input, weight, bias, position.contiguous(), num_head, dim_head, dim_position)

    @staticmethod
    def backward(ctx, grad_out):
        input, weight, bias = ctx.saved_tensors
        dx, dW, db, _, _ = ops.projpos_backward(input, weight, bias, None, grad_out.contiguous(), 0.0, *ctx.dims)
        return dx, dW, (db if bias is not None else None), None, None, None, None


class Multihead_Porjection_Layernorm_with_Position_Function(torch.autograd.Function):
    """Autograd wrapper with the reference's class name (extension/bind/galerkin_attention.py:37-65)."""

    @staticmethod
    def forward(ctx, input, weight, bias, ln_weight, ln_bias, position, norm_eps, num_head, dim_head, dim_position):
        input, weight = input.contiguous(), weight.contiguous()
        ctx.save_for_backward(input, weight, bias, ln_weight.contiguous())
        ctx.args = (norm_eps, num_head, dim_head, dim_position)
        return ops.projpos_lnorm(input, weight, bias, ln_weight.contiguous(), ln_bias.contiguous(), position.contiguous(),
                                 norm_eps, num_head, dim_head, dim_position)

    @staticmethod
    def backward(ctx, grad_out):
        input, weight, bias, ln_weight = ctx.saved_tensors
        dx, dW, db, dlnw, dlnb = ops.projpos_backward(input, weight, bias, ln_weight, grad_out.contiguous(), *ctx.args)
        return dx, dW, (db if bias is not None else None), dlnw, dlnb, None, None, None, None, None


def multihead_projection_with_position_rrc_cuda(
    input: Tensor, weight: Tensor, bias: Tensor, position: Tensor, num_head, dim_head, dim_position
) -> Tensor:
    """[B,S,D] -> [B, num_head, dim_position + dim_head, S]; computes input @ weight (weight used as [k][n]);
    differentiable in input, weight and bias."""
    if _needs_grad(input, weight, bias):
        return Multihead_Porjection_with_Position_Function.apply(input, weight, bias, position, num_head, dim_head, dim_position)
    return ops.projpos(input, weight, bias, position, num_head, dim_head, dim_position)


def multihead_projection_layernorm_with_position_rrc_cuda(
    input: Tensor, weight: Tensor, bias: Tensor, ln_weight: Tensor, ln_bias: Tensor, position: Tensor,
    norm_eps, num_head, dim_head, dim_position
) -> Tensor:
    """As above with a LayerNorm over each head's channels; position rows are not normalised; differentiable in input,
    weight, bias, ln_weight and ln_bias."""
    if _needs_grad(input, weight, bias, ln_weight, ln_bias):
        return Multihead_Porjection_Layernorm_with_Position_Function.apply(
            input, weight, bias, ln_weight, ln_bias, position, norm_eps, num_head, dim_head, dim_position)
    return ops.projpos_lnorm(input, weight, bias, ln_weight, ln_bias, position, norm_eps, num_head, dim_head, dim_position)


class Multihead_Galerkin_Attention_cccr_Function(torch.autograd.Function):
    """Autograd wrapper with the reference's class name (extension/bind/galerkin_attention.py:68-84)."""

    @staticmethod
    def forward(ctx, Q: Tensor, K: Tensor, V: Tensor) -> Tensor:
        Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
        ctx.save_for_backward(Q, K, V)
        return ops.galerkin_attention(Q, K, V)

    @staticmethod
    def backward(ctx, grad_attn: Tensor):
        Q, K, V = ctx.saved_tensors
        return ops.galerkin_attention_backward(Q, K, V, grad_attn.contiguous())


def multihead_galerkin_attention_cccr_cuda(Q: Tensor, K: Tensor, V: Tensor) -> Tensor:
    """Q,K,V [B,H,d_posk,S] -> [B,H,S,d_posk] = Q^T (K V^T / S); differentiable in Q, K and V."""
    if _needs_grad(Q, K, V):
        return Multihead_Galerkin_Attention_cccr_Function.apply(Q, K, V)
    return ops.galerkin_attention(Q, K, V)


def batched_skinny_gemm(A: Tensor, B: Tensor, alpha: float = 1.0) -> Tensor:
    """[...,M,K] @ [...,K,N] * alpha with K the long dimension."""
    return ops.batched_skinny_gemm(A, B, alpha)
