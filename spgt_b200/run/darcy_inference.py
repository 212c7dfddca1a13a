"""Single-GPU validation run on real Darcy data: the counterpart of the reference's run/darcy_inference.py:14-64.

The training file supplies the node / target normalisers, the validation file the samples; the model takes
checkpoint['Module'] (SpGT state-dict keys).  Every batch goes host -> device -> forward -> metric; the metric is the
mean over batches of the per-batch mean relative L2 (engine/darcy_engine.py:33-46, metric_reduction 'L1').
"""
import time
from typing import Optional

import torch

from ..dataset.darcy_dataset import DarcyDataset, GaussNormalizer
from ..engine.darcy_engine import HostInference
from ..engine.metric import relative_l2_metric
from ..network.sp_model import Sp_GalerkinTransformer2D


def get_gauss_normalizer(train_path: str, sub_node: int):
    """Normalisers fitted on the training file at the given sub-sampling (dataset/darcy_dataset.py of the reference)."""
    ds = DarcyDataset(train_path, sub_node, is_training=True)
    return ds.node_normalizer, ds.target_normalizer


def validate_epoch_darcy(model, dataset: DarcyDataset, batch_size: int, device, use_graphs: bool = False) -> float:
    """Mean over batches of the per-batch metric, as the reference's validate_epoch_darcy computes it."""
    engine = HostInference(model, device, use_graphs=use_graphs)
    batches = list(dataset.batches(batch_size, pin_memory=True))
    total, full = 0.0, batches[0]['node'].shape[0]
    with torch.no_grad():
        # a ragged last batch has another shape: run it eagerly after the full ones
        regular = [b for b in batches if b['node'].shape[0] == full]
        preds = engine.run(regular)
        for b, p in zip(regular, preds):
            total += float(relative_l2_metric(p.to(device), b['target'].to(device)))
        for b in batches[len(regular):]:
            p = model(b['node'].to(device), b['position'].to(device), b['grid'].to(device))
            total += float(relative_l2_metric(p, b['target'].to(device)))
    from .. import ops
    ops.check_tc_status('validate_epoch_darcy')
    return total / len(batches)


def darcy_inference(cfg: dict, checkpoint: Optional[dict], train_path: str, valid_path: str, device='cuda:0',
                    use_graphs: bool = False) -> float:
    device = torch.device(device)
    torch.cuda.set_device(device)
    node_normalizer, target_normalizer = get_gauss_normalizer(train_path, cfg['subsample_node'])
    valid_ds = DarcyDataset(valid_path, cfg['subsample_node'], cfg['subsample_attn'], cfg.get('num_data'),
                            cfg.get('fine_resolution'), is_training=False, noise=cfg.get('noise', 0.0),
                            random_seed=cfg.get('seed', 1127802), node_normalizer=node_normalizer)
    cfg = dict(cfg)
    cfg['target_normalizer'] = (target_normalizer or GaussNormalizer()).numpy_to_torch(device)
    model = Sp_GalerkinTransformer2D(cfg)
    if checkpoint is not None:
        model.load_state_dict(checkpoint['Module'])
    model = model.to(device).eval()
    t0 = time.time()
    metric = validate_epoch_darcy(model, valid_ds, 2 * cfg['batch_size'], device, use_graphs)
    print(f'========== valid_time: {time.time() - t0:.6f} ==========')
    print(f'========== Metric : {metric} ==========')
    return metric
