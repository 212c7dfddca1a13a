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


class WeightedL2Loss2D(torch.nn.Module):
    """Training loss / validation metric of the reference (engine/metric.py:5-93), same constructor and return values.

    forward(pred, target, pred_grad, target_grad, coeff) -> (loss, regularizer, metric) for [N, r, r, 1] fields:
      e_n   = beta * mean((p - t)^2) / (mean(t^2) + eps)                      (+ alpha * the coefficient-weighted H1 term
                                                                               when alpha > 0 and pred_grad is given)
      loss  = mean_n sqrt(e_n)   (is_normalization)  or  mean_n e_n
      metric: 'L1' mean_n sqrt(e_n), 'L2' sqrt(mean_n e_n), 'Linf' max_n sqrt(e_n)
      regularizer (is_regularization and target_grad given): gamma * H * mean((coeff * (target_grad - D pred))^2) over the
      interior / (dim * mean(coeff * target_grad^2) + eps), D = central differences with the given dilation scaled by S,
      reduced like the loss; otherwise a zero."""

    def __init__(self, S, dim=2, dilation=2, alpha=0.0, beta=1.0, gamma=0.1, delta=0.0, eps=1.0e-10,
                 is_regularization=False, is_normalization=True, metric_reduction='L1') -> None:
        super().__init__()
        self.S, self.H, self.dim, self.dilation = S, 1.0 / S, dim, dilation
        self.alpha, self.beta, self.gamma, self.delta, self.eps = alpha, beta, gamma, delta * (1.0 / S) ** dim, eps
        self.is_regularization, self.is_normalization, self.metric_reduction = is_regularization, is_normalization, metric_reduction

    def _central_diff(self, X: torch.Tensor, S: int) -> torch.Tensor:
        d, s = self.dilation, self.dilation // 2
        gx = (X[:, d:, s:-s] - X[:, :-d, s:-s]) / d
        gy = (X[:, s:-s, d:] - X[:, s:-s, :-d]) / d
        return torch.stack([gx, gy], dim=-1) * S

    def forward(self, pred, target, pred_grad=None, target_grad=None, coeff=None):
        pred, target = pred.squeeze(dim=-1), target.squeeze(dim=-1)
        target_norm = target.pow(2).mean(dim=[1, 2]) + self.eps
        grad_norm = self.dim * (coeff * target_grad.pow(2)).mean(dim=[1, 2, 3]) + self.eps if target_grad is not None else 1
        err = self.beta * (pred - target).pow(2).mean(dim=[1, 2]) / target_norm
        if self.alpha > 0 and pred_grad is not None:
            err = err + self.alpha * (coeff * (pred_grad - target_grad)).pow(2).mean(dim=[1, 2, 3]) / grad_norm
        if self.metric_reduction == 'L2':
            metric = err.mean().sqrt()
        elif self.metric_reduction == 'Linf':
            metric = err.sqrt().max()
        else:
            metric = err.sqrt().mean()
        loss = err.sqrt().mean() if self.is_normalization else err.mean()
        if self.is_regularization and target_grad is not None:
            s = self.dilation // 2
            diff = coeff[:, s:-s, s:-s] * (target_grad[:, s:-s, s:-s, :] - self._central_diff(pred, self.S))
            reg = self.gamma * self.H * diff.pow(2).mean(dim=[1, 2, 3]) / grad_norm
            reg = reg.sqrt().mean() if self.is_normalization else reg.mean()
        else:
            reg = torch.zeros(1, device=loss.device, requires_grad=loss.requires_grad)
        return loss, reg, metric
