"""Drop-in for the reference's extension/bind/datamove.py (forward / inference only):
same names and signatures as extension/bind/datamove.py:68-87."""
from torch import Tensor

from ... import ops


def batched_transpose(X: Tensor, batch_list: list, M_list: list, N_list: list) -> Tensor:
    """[batch..., M..., N...] -> [batch..., N..., M...]."""
    return ops.batched_transpose(X, batch_list, M_list, N_list)


def transpose_gather_dual(src: Tensor, dim_list: list, H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2):
    """complex64 [dim..., H_all, W_all] -> two [H_low, W_low, dim...] blocks."""
    return ops.transpose_gather_dual(src, dim_list, H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2)


def transpose_scatter_dual(src1: Tensor, src2: Tensor, dim_list: list, H_all, W_all, H_low, W_low,
                           H_base_1, W_base_1, H_base_2, W_base_2) -> Tensor:
    """Inverse of transpose_gather_dual; everything outside the two blocks is zero."""
    return ops.transpose_scatter_dual(src1, src2, dim_list, H_all, W_all, H_low, W_low, H_base_1, W_base_1, H_base_2, W_base_2)
