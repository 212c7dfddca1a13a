"""Single-GPU training run on Darcy data: the counterpart of the reference's run/darcy_train.py:16-87.

Adam + OneCycleLR (pct_start 0.3, div_factor = final_div_factor = 1e4), loss = relative L2 + the gradient regulariser
with weight cfg['metric_gamma'], validation metric = relative L2 on the fused inference path, best state kept.
`train_data` / `valid_data` are .mat paths or dicts holding the arrays 'a' and 'u' (e.g. from dataset.darcy_generate).
"""
import time
from typing import Optional

import torch

from ..dataset.darcy_dataset import DarcyDataset
from ..engine.metric import WeightedL2Loss2D
from ..engine.train import run_train
from ..network.sp_model import Sp_GalerkinTransformer2D


def darcy_train(cfg: dict, train_data, valid_data, device='cuda:0', num_valid: Optional[int] = 128, log=print) -> dict:
    device = torch.device(device)
    torch.cuda.set_device(device)
    torch.manual_seed(cfg['seed'])
    sub_node, sub_attn = cfg['subsample_node'], cfg['subsample_attn']
    train_ds = DarcyDataset(train_data, sub_node, sub_attn, cfg.get('num_data'), cfg.get('fine_resolution'), is_training=True,
                            noise=cfg.get('noise', 0.0), random_seed=cfg['seed'])
    valid_ds = DarcyDataset(valid_data, sub_node, sub_attn, num_valid, cfg.get('fine_resolution'), is_training=False,
                            noise=cfg.get('noise', 0.0), random_seed=cfg['seed'], node_normalizer=train_ds.node_normalizer)
    cfg = dict(cfg)
    cfg['target_normalizer'] = train_ds.target_normalizer.numpy_to_torch(device)
    model = Sp_GalerkinTransformer2D(cfg).to(device)
    epochs, lr, bs = cfg['epochs'], cfg['lr'], cfg['batch_size']
    steps_per_epoch = (len(train_ds) + bs - 1) // bs
    optimizer = torch.optim.Adam(model.parameters(), lr=lr)
    scheduler = torch.optim.lr_scheduler.OneCycleLR(optimizer, max_lr=lr, epochs=epochs, steps_per_epoch=steps_per_epoch,
                                                    pct_start=0.3, div_factor=1e4, final_div_factor=1e4)
    r = cfg['r_node']
    train_loss = WeightedL2Loss2D(is_regularization=True, S=r, gamma=cfg['metric_gamma'])
    valid_loss = WeightedL2Loss2D(is_regularization=False, S=r)
    gen = torch.Generator().manual_seed(cfg['seed'])

    def train_batches():                                      # shuffled every epoch, as the reference's DataLoader(shuffle=True)
        order = torch.randperm(len(train_ds), generator=gen).tolist()
        for s in range(0, len(order), bs):
            items = [train_ds[i] for i in order[s:s + bs]]
            yield {k: torch.stack([it[k] for it in items]) for k in items[0]}

    t0 = time.time()
    checkpoint = run_train(model, train_batches, lambda: valid_ds.batches(2 * bs), train_loss, valid_loss, optimizer, scheduler,
                           epochs=epochs, patience=20, device=device, log=log)
    if log is not None:
        log(f'========== train_time: {time.time() - t0:.6f} ==========')
    checkpoint['Train_Config'] = {k: v for k, v in cfg.items() if k != 'target_normalizer'}
    return checkpoint
