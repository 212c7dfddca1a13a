"""Batch-sharded multi-GPU Darcy inference (reference: run/ddp_darcy_inference.py:15-72).

One process per GPU (torchrun).  Every sample is independent through the whole forward, so the global sample
range is cut into one contiguous slice per rank and there is no collective inside the forward; NCCL is used only
after the last batch, to gather the predictions and to sum the metric.  (The reference wraps the model in
DistributedDataParallel, whose only effect at inference is a parameter broadcast at construction; here every
rank builds identical weights from the same seed or loads the same checkpoint.)

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m spgt_b200.run.ddp_darcy_inference
"""
import os
import time
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [begin, end) of rank; sizes differ by at most one and earlier ranks get the larger ones."""
    base, extra = divmod(n_total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def distributed_initialize(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """env:// rendezvous from RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*; returns (rank, world, local_rank).
    Single-process runs (no RANK in the environment) do not create a process group."""
    if 'RANK' not in os.environ:
        return 0, 1, 0
    rank, world, local = int(os.environ['RANK']), int(os.environ['WORLD_SIZE']), int(os.environ.get('LOCAL_RANK', 0))
    if not dist.is_initialized():
        backend = backend or ('nccl' if torch.cuda.is_available() else 'gloo')
        if backend == 'nccl':
            torch.cuda.set_device(local)
        dist.init_process_group(backend=backend, init_method='env://')
    return rank, world, local


def gather_predictions(local_pred: torch.Tensor, n_total: int, rank: int, world: int) -> torch.Tensor:
    """All ranks obtain [n_total, ...] in global sample order from their contiguous slices (sizes may differ by 1)."""
    if world == 1:
        return local_pred
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    counts = [e - b for b, e in sizes]
    if len(set(counts)) == 1:
        out = torch.empty((n_total, *local_pred.shape[1:]), dtype=local_pred.dtype, device=local_pred.device)
        dist.all_gather_into_tensor(out, local_pred.contiguous())
        return out
    # uneven slices: pad every rank's block to the largest count (collectives need equal sizes), then trim
    cmax = max(counts)
    padded = torch.zeros((cmax, *local_pred.shape[1:]), dtype=local_pred.dtype, device=local_pred.device)
    padded[:local_pred.shape[0]] = local_pred
    out = torch.empty((world * cmax, *local_pred.shape[1:]), dtype=local_pred.dtype, device=local_pred.device)
    dist.all_gather_into_tensor(out, padded)
    return torch.cat([out[r * cmax:r * cmax + c] for r, c in enumerate(counts)], dim=0)


def reduce_metric(metric_sum: torch.Tensor, count: torch.Tensor, world: int) -> float:
    """Global mean of the per-sample metric from per-rank (sum, count)."""
    packed = torch.stack([metric_sum.reshape(()).double(), count.reshape(()).double()])
    if world > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM)
    return float(packed[0] / packed[1].clamp_min(1.0))


class ShardedGather:
    """`post` hook of HostInference for a rank of a sharded run: after the forward of the rank's slice of a global batch it
    gathers all ranks' predictions into the global batch (one all_gather_into_tensor) and sums the per-sample metric over
    all ranks (one all_reduce of (sum, count)), both on the compute stream.  What the host loop downloads per batch:
    download='predictions': rank 0 the gathered predictions, the other ranks the reduced (sum, count);
    download='metric': every rank the reduced (sum, count) only, as the reference's driver reads back nothing but the metric
    (run/ddp_darcy_inference.py:62, engine/darcy_engine.py:33-46); the gathered predictions of the last batch stay on the
    device in `last_full`.  `metric(i)` gives the global mean of batch i afterwards.
    The global batch must split evenly over the ranks (collectives need equal block sizes)."""

    def __init__(self, n_total: int, rank: int, world: int, sample_shape, device, download: str = 'predictions'):
        if n_total % world != 0:
            raise ValueError('ShardedGather needs a global batch that is a multiple of the number of ranks')
        if download not in ('predictions', 'metric'):
            raise ValueError("download must be 'predictions' or 'metric'")
        self.n_total, self.rank, self.world, self.download = n_total, rank, world, download
        self.last_full = None
        self.full = [torch.empty((n_total, *sample_shape), dtype=torch.float32, device=device) for _ in range(2)] if world > 1 else None
        self.packed = [torch.zeros(2, dtype=torch.float64, device=device) for _ in range(2)]
        self.packed_host = {}

    def __call__(self, pred: torch.Tensor, slot: Dict[str, torch.Tensor], i: int) -> torch.Tensor:
        # Everything here is enqueued on the compute stream without a host synchronisation (no Python scalars are
        # turned into device tensors): the host loop must stay ahead of the device to overlap the next upload.
        from ..engine.metric import relative_l2_per_sample
        packed = self.packed[i & 1]
        if 'target' in slot:
            packed[0:1].copy_(relative_l2_per_sample(pred, slot['target']).sum().reshape(1))
            packed[1:2].fill_(float(pred.shape[0]))
        if self.world > 1:
            full = self.full[i & 1]
            dist.all_gather_into_tensor(full, pred.contiguous())
            dist.all_reduce(packed, op=dist.ReduceOp.SUM)
        else:
            full = pred
        if i not in self.packed_host:
            self.packed_host[i] = torch.empty(2, dtype=torch.float64, pin_memory=pred.is_cuda)
        self.packed_host[i].copy_(packed, non_blocking=True)
        self.last_full = full
        return full if (self.rank == 0 and self.download == 'predictions') else packed

    def metric(self, i: int) -> float:
        """Global mean of the per-sample metric of batch i (valid once the run has returned)."""
        p = self.packed_host[i]
        return float(p[0] / max(float(p[1]), 1.0))


def run_sharded(forward: Callable[[Dict[str, torch.Tensor]], torch.Tensor], make_batch: Callable[[range], Dict[str, torch.Tensor]],
                n_total: int, batch_size: int, rank: int, world: int, target_fn: Optional[Callable] = None,
                sample_shape: Optional[Tuple[int, ...]] = None, device=None):
    """Evaluate samples [0, n_total) sharded over ranks.  `make_batch(range)` builds the inputs of global sample
    indices, `forward(batch)` returns predictions [n, ...].  Returns (all predictions in global order, metric or None).

    Every rank enters both collectives, also one whose slice is empty (n_total < world): it contributes a [0, ...]
    block and a zero (sum, count).  Such a rank cannot learn the per-sample shape from a prediction of its own, so
    callers that may shard fewer samples than ranks pass `sample_shape` (and `device`)."""
    from ..engine.metric import relative_l2_sums
    begin, end = shard_range(n_total, rank, world)
    preds, msum, cnt = [], None, None
    for b0 in range(begin, end, batch_size):
        idx = range(b0, min(b0 + batch_size, end))
        batch = make_batch(idx)
        pred = forward(batch)
        preds.append(pred)
        if target_fn is not None:
            s, c = relative_l2_sums(pred, target_fn(idx, batch))
            msum = s if msum is None else msum + s
            cnt = c if cnt is None else cnt + c
    if preds:
        local = torch.cat(preds, dim=0)
    else:
        if sample_shape is None:
            raise ValueError(f'rank {rank} has no samples (n_total={n_total}, world={world}): pass sample_shape so that it '
                             'can still take part in the gather')
        local = torch.empty((0, *sample_shape), dtype=torch.float32, device=device)
    full = gather_predictions(local, n_total, rank, world)
    metric = None
    if target_fn is not None:
        if msum is None:
            msum = torch.zeros((), dtype=torch.float32, device=local.device)
            cnt = torch.zeros((), dtype=torch.float32, device=local.device)
        metric = reduce_metric(msum, cnt, world)
    if local.is_cuda:
        from .. import ops
        ops.check_tc_status('run_sharded')
    return full, metric


def darcy_inference_ddp(cfg: dict, checkpoint: Optional[dict] = None, num_samples: int = 64, seed: int = 4):
    """Synthetic-field stand-in for the reference driver: build the model (checkpoint['Module'] if given, else
    seeded random init), shard `num_samples` synthetic coefficient fields over the ranks in batches of
    2 * cfg['batch_size'] (as the reference's DataLoader does), gather predictions."""
    from ..dataset.darcy_dataset import GaussNormalizer, synthetic_darcy_batch
    from ..network.sp_model import Sp_GalerkinTransformer2D
    rank, world, local = distributed_initialize()
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    cfg = dict(cfg)
    cfg.setdefault('target_normalizer', GaussNormalizer())
    torch.manual_seed(seed)
    model = Sp_GalerkinTransformer2D(cfg)
    if checkpoint is not None:
        model.load_state_dict(checkpoint['Module'])
    model = model.to(device).eval()

    def make_batch(idx):
        data = synthetic_darcy_batch(idx, cfg['fine_resolution'], cfg['subsample_node'], cfg['subsample_attn'], seed)
        return {k: v.to(device, non_blocking=True) for k, v in data.items()}

    t0 = time.time()
    r = cfg['r_node']
    pred, _ = run_sharded(lambda b: model(b['node'], b['position'], b['grid']), make_batch, num_samples,
                          2 * cfg['batch_size'], rank, world, sample_shape=(r, r, 1), device=device)
    torch.cuda.synchronize()
    if rank == 0:
        print(f'========== valid_time: {time.time() - t0:.6f} ==========')
        print(f'========== predictions: {tuple(pred.shape)} on {world} rank(s) ==========')
    return pred


if __name__ == '__main__':
    from ..config.config_accessor import get_darcy_config
    darcy_inference_ddp(get_darcy_config(2, 8, num_frequence_mode=12))
    if dist.is_initialized():
        dist.destroy_process_group()
