"""Training loop of the reference (engine/train.py:13-76, engine/darcy_engine.py:9-29) on this package's model.

The model's training-mode forward is the differentiable path (this library's attention / projection / data-movement
ops with their backward kernels, library ops under torch autograd for the rest); validation runs the fused inference
kernels.  Batches are dicts as DarcyDataset.batches() yields them.
"""
from typing import Callable, Iterable, Optional

import torch


def train_epoch_darcy(model: torch.nn.Module, train_batches: Iterable[dict], train_loss_func: Callable, optimizer,
                      lr_scheduler=None, grad_clip: float = 0.99, *, device) -> torch.Tensor:
    """One pass over the training batches: loss + regulariser, backward, gradient clipping, optimizer (and per-batch
    scheduler) step.  Returns the mean loss of the epoch as a tensor."""
    model.train()
    total, n = torch.zeros(1, device=device), 0
    for data in train_batches:
        node, position, grid = (data[k].to(device, non_blocking=True) for k in ('node', 'position', 'grid'))
        coeff, target, target_grad = (data[k].to(device, non_blocking=True) for k in ('coeff', 'target', 'target_grad'))
        optimizer.zero_grad(set_to_none=True)
        pred = model(node, position, grid)
        loss, reg, _ = train_loss_func(pred, target, pred_grad=None, target_grad=target_grad, coeff=coeff)
        loss = loss + reg
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), grad_clip)
        optimizer.step()
        if lr_scheduler is not None:
            lr_scheduler.step()
        total, n = total + loss.detach(), n + 1
    return total / max(n, 1)


def validate_epoch(model: torch.nn.Module, valid_batches: Iterable[dict], valid_loss_func: Callable, *, device) -> torch.Tensor:
    """Mean over batches of the validation metric, on the fused inference path (engine/darcy_engine.py:33-46)."""
    model.eval()
    total, n = torch.zeros(1, device=device), 0
    with torch.no_grad():
        for data in valid_batches:
            pred = model(data['node'].to(device), data['position'].to(device), data['grid'].to(device))
            _, _, metric = valid_loss_func(pred, data['target'].to(device), pred_grad=None, target_grad=None, coeff=None)
            total, n = total + metric, n + 1
    return total / max(n, 1)


_EPOCH_SCHEDULERS = ('ReduceLROnPlateau', 'StepLR', 'MultiplicativeLR', 'MultiStepLR', 'ExponentialLR', 'LambdaLR')


def run_train(model: torch.nn.Module, train_batches: Callable[[], Iterable[dict]], valid_batches: Callable[[], Iterable[dict]],
              train_loss_func: Callable, valid_loss_func: Callable, optimizer, lr_scheduler, grad_clip: float = 0.999,
              epochs: int = 10, start_epoch: int = 0, patience: Optional[int] = None, *, device, log: Callable = None) -> dict:
    """Epoch loop with the reference's bookkeeping: loss / metric history, the best epoch's state_dict under 'Module',
    early stopping after `patience` epochs without improvement, schedulers stepped per epoch or per batch by their kind.
    `train_batches` / `valid_batches` are callables that return a fresh iterable of batches for an epoch."""
    per_epoch = any(name in type(lr_scheduler).__name__ for name in _EPOCH_SCHEDULERS) if lr_scheduler is not None else True
    patience = epochs if patience is None else patience
    best_metric, stall = float('inf'), 0
    checkpoint = dict(loss_history=[], metric_history=[])
    for epoch in range(start_epoch, start_epoch + epochs):
        loss = float(train_epoch_darcy(model, train_batches(), train_loss_func, optimizer,
                                       None if per_epoch else lr_scheduler, grad_clip, device=device))
        metric = float(validate_epoch(model, valid_batches(), valid_loss_func, device=device))
        checkpoint['loss_history'].append(loss)
        checkpoint['metric_history'].append(metric)
        if per_epoch and lr_scheduler is not None:
            if 'ReduceLROnPlateau' in type(lr_scheduler).__name__:
                lr_scheduler.step(metric)
            else:
                lr_scheduler.step()
        if metric < best_metric:
            best_metric, stall = metric, 0
            checkpoint.update(Best_Epoch=epoch, Best_Metric=metric,
                              Module={k: v.detach().clone() for k, v in model.state_dict().items()})
        else:
            stall += 1
        if log is not None:
            log(f'epoch {epoch + 1}: loss {loss:.3e} | metric {metric:.3e} | best {best_metric:.3e} | lr {optimizer.param_groups[0]["lr"]:.3e}')
        if stall > patience:
            break
    return checkpoint
