"""Relative L2 metric of the reference's validation loop (engine/metric.py:47-67, metric_reduction='L1')."""
import torch


def relative_l2_per_sample(pred: torch.Tensor, target: torch.Tensor, eps: float = 1.0e-10) -> torch.Tensor:
    """sqrt(mean((p - t)^2) / (mean(t^2) + eps)) per sample for [N, r, r, 1] tensors: one CUDA kernel on device
    tensors (spgt_relative_l2_fwd); host tensors (the gloo tests of the sharding logic) use the same formula in torch."""
    if pred.is_cuda:
        from .. import ops
        return ops.relative_l2(pred, target, eps)
    p, t = pred.squeeze(-1), target.squeeze(-1)
    return ((p - t).pow(2).mean(dim=[1, 2]) / (t.pow(2).mean(dim=[1, 2]) + eps)).sqrt()


def relative_l2_metric(pred: torch.Tensor, target: torch.Tensor, eps: float = 1.0e-10) -> torch.Tensor:
    """The reference's metric with metric_reduction='L1': mean over samples of the per-sample relative L2."""
    return relative_l2_per_sample(pred, target, eps).mean()


def relative_l2_sums(pred: torch.Tensor, target: torch.Tensor, eps: float = 1.0e-10):
    """(sum over samples of the per-sample relative L2, number of samples): what ranks all-reduce."""
    e = relative_l2_per_sample(pred, target, eps)
    return e.sum(), torch.tensor(float(e.shape[0]), device=e.device)
