"""Relative L2 metric of the reference's validation loop (engine/metric.py:47-67, metric_reduction='L1')."""
import torch


def relative_l2_metric(pred: torch.Tensor, target: torch.Tensor, eps: float = 1.0e-10) -> torch.Tensor:
    """mean over samples of sqrt(mean((p - t)^2) / (mean(t^2) + eps)) for [N, r, r, 1] tensors."""
    p, t = pred.squeeze(-1), target.squeeze(-1)
    loss = (p - t).pow(2).mean(dim=[1, 2]) / (t.pow(2).mean(dim=[1, 2]) + eps)
    return loss.sqrt().mean()


def relative_l2_sums(pred: torch.Tensor, target: torch.Tensor, eps: float = 1.0e-10):
    """(sum over samples of the per-sample relative L2, number of samples): what ranks all-reduce."""
    p, t = pred.squeeze(-1), target.squeeze(-1)
    loss = (p - t).pow(2).mean(dim=[1, 2]) / (t.pow(2).mean(dim=[1, 2]) + eps)
    return loss.sqrt().sum(), torch.tensor(float(p.shape[0]), device=p.device)
