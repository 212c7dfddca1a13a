"""Sharding, gather and metric reduction of the multi-GPU driver, run as 2 gloo ranks on CPU."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spgt_b200.run.ddp_darcy_inference import shard_range


def test_shard_range_partitions_exactly():
    for n, w in ((64, 8), (64, 1), (10, 4), (3, 8), (0, 2)):
        spans = [shard_range(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def _worker(rank, world, port, n_total, batch, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    from spgt_b200.run.ddp_darcy_inference import distributed_initialize, run_sharded
    r, w, _ = distributed_initialize('gloo')
    assert (r, w) == (rank, world)

    def make_batch(idx):
        return {'node': torch.tensor([[float(i)] for i in idx]).view(-1, 1, 1, 1).expand(-1, 3, 3, 1).contiguous()}

    forward = lambda b: b['node'] * 2.0 + 1.0                     # stands in for the model: sample i -> 2 i + 1
    target = lambda idx, b: b['node'] * 2.0 + 1.5                  # constant offset -> known relative error
    pred, metric = run_sharded(forward, make_batch, n_total, batch, r, w, target_fn=target, sample_shape=(3, 3, 1))
    torch.save({'pred': pred, 'metric': metric}, os.path.join(out_dir, f'rank{rank}.pt'))
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _run(n_total, batch, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_total, batch, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f'rank{r}.pt')) for r in range(world)]
    expect = (torch.arange(n_total, dtype=torch.float32) * 2 + 1).view(-1, 1, 1, 1).expand(-1, 3, 3, 1)
    ref_metric = float((0.5 / (torch.arange(n_total, dtype=torch.float64) * 2 + 1.5)).mean())
    for r in res:
        assert torch.equal(r['pred'], expect)                      # every rank holds all samples, in global order
        assert abs(r['metric'] - ref_metric) < 1e-6
    return res


def test_two_ranks_even_split(tmp_path):
    _run(8, 3, tmp_path)


def test_two_ranks_uneven_split(tmp_path):
    _run(7, 2, tmp_path)


def test_two_ranks_one_sample(tmp_path):
    """Fewer samples than ranks: the rank with an empty slice still enters the gather and the metric reduction."""
    _run(1, 2, tmp_path)


def _gather_worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    from spgt_b200.run.ddp_darcy_inference import ShardedGather, distributed_initialize, shard_range
    r, w, _ = distributed_initialize('gloo')
    n_total = 6
    b, e = shard_range(n_total, r, w)
    gather = ShardedGather(n_total, r, w, (3, 3, 1), 'cpu')
    outs = []
    for step in range(3):                                   # three steps: the two internal buffers are reused
        pred = (torch.arange(b, e, dtype=torch.float32) + 10 * step).view(-1, 1, 1, 1).expand(-1, 3, 3, 1).contiguous()
        slot = {'target': pred + 0.5}
        outs.append(gather(pred, slot, step).clone())
    # metric-only download (what the reference's driver reads back): every rank gets the reduced (sum, count), the gathered
    # predictions stay in `last_full`
    gm = ShardedGather(n_total, r, w, (3, 3, 1), 'cpu', download='metric')
    pred = torch.arange(b, e, dtype=torch.float32).view(-1, 1, 1, 1).expand(-1, 3, 3, 1).contiguous()
    got = gm(pred, {'target': pred + 0.5}, 0).clone()
    torch.save({'outs': outs, 'metrics': [gather.metric(i) for i in range(3)], 'metric_only': got, 'last_full': gm.last_full.clone(),
                'metric_only_value': gm.metric(0)}, os.path.join(out_dir, f'g{rank}.pt'))
    dist.destroy_process_group()


def test_sharded_gather_hook_two_ranks(tmp_path):
    """The post-forward hook of the host loop: rank 0 receives the global batch in order, the others the reduced metric sums."""
    world = 2
    mp.spawn(_gather_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f'g{r}.pt')) for r in range(world)]
    for step in range(3):
        expect = (torch.arange(6, dtype=torch.float32) + 10 * step).view(-1, 1, 1, 1).expand(-1, 3, 3, 1)
        assert torch.equal(res[0]['outs'][step], expect)
        ref_metric = float((0.5 / (torch.arange(6, dtype=torch.float64) + 10 * step + 0.5)).mean())
        assert res[1]['outs'][step].shape == (2,) and abs(float(res[1]['outs'][step][0] / res[1]['outs'][step][1]) - ref_metric) < 1e-6
        for r in range(world):
            assert abs(res[r]['metrics'][step] - ref_metric) < 1e-6
    ref0 = float((0.5 / (torch.arange(6, dtype=torch.float64) + 0.5)).mean())
    for r in range(world):
        assert res[r]['metric_only'].shape == (2,) and float(res[r]['metric_only'][1]) == 6.0
        assert abs(res[r]['metric_only_value'] - ref0) < 1e-6
        assert torch.equal(res[r]['last_full'], torch.arange(6, dtype=torch.float32).view(-1, 1, 1, 1).expand(-1, 3, 3, 1))
