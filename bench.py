#!/usr/bin/env python
"""Darcy Galerkin Transformer inference benchmark (211 x 211 fine grid, 53 x 53 attention grid).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One rank per GPU (torchrun for N > 1).  A step is one forward of the full model over this rank's batch of
synthetic Darcy coefficient fields; rank 0 prints one JSON line.  `value` is samples/s with the inputs resident
in HBM, `e2e` the same metric through the host-facing API with pinned host buffers (upload and download inside
the timed region), `roofline` the Galerkin attention kernel's achieved HBM bandwidth measured with CUDA events
around its launches inside the timed steps, `cpu_baseline` the CPU oracle (a port of the reference's own CPU
path) on a bounded sample.  `--impl reference` times that CPU path alone with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = 'darcy_gt_inference_samples_per_s_211'
FINE, SUB_NODE, SUB_ATTN, MODES, SEED = 421, 2, 8, 12, 4
# DRAM bytes (read + write) of one galerkin_attn_tc_kernel launch at B=64, H=4, S=2809 from the ncu capture
# summarised in profiles/ (None until a capture of the current kernel exists).
ATTN_TRAFFIC_BYTES = 342_400_000   # dram read + write per launch from the ncu capture under profiles/ (342.1 - 342.6 MB)


def measured_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return 6650.0, 'fallback'


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs (read-only query)."""
    Q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '200',
                                          '-i', str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith('active'):
                    reasons.add(n)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2], 'sm_max_mhz': max(mx), 'reasons': sorted(reasons), 'samples': len(sm)}


def oracle_setup(batch: int, seed: int = SEED):
    from oracle import gt_oracle as O
    from spgt_b200.dataset.darcy_dataset import synthetic_darcy_batch
    cfg = O.default_config(FINE, SUB_NODE, SUB_ATTN, MODES)
    data = synthetic_darcy_batch(range(batch), FINE, SUB_NODE, SUB_ATTN, seed)
    return O, cfg, data


def oracle_params(seed: int = SEED):
    """Random-init weights of the benchmark architecture in the SpGT layout (same construction as the GPU model)."""
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    torch.manual_seed(seed)
    model = Sp_GalerkinTransformer2D(get_darcy_config(SUB_NODE, SUB_ATTN, num_frequence_mode=MODES))
    return {k: v.detach().clone() for k, v in model.state_dict().items()}


WORKLOAD = ('full Darcy Galerkin Transformer forward, fine grid 211x211, attention grid 53x53, 6 encoder '
            'layers (hidden 128, 4 heads, FFN 256), FNO2d regressor (2 spectral layers, width 32, 12 modes)')


def use_all_host_threads() -> int:
    """The launcher of multi-rank runs exports OMP_NUM_THREADS=1; the CPU legs use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def time_oracle(sample_batch: int, steps: int, warmup: int):
    O, cfg, data = oracle_setup(sample_batch)
    p = oracle_params()
    fwd = lambda: O.model_forward(data['node'], data['position'], data['grid'], p, cfg)
    with torch.no_grad():
        for _ in range(warmup):
            fwd()
        t0 = time.perf_counter()
        for _ in range(steps):
            fwd()
        dt = time.perf_counter() - t0
    return sample_batch * steps / dt, dt / steps


def run_reference(args, rank):
    if rank != 0:
        return
    cores = use_all_host_threads()
    sample = 8
    sps, per_step = time_oracle(sample, args.steps, args.warmup)
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': sps, 'unit': 'samples/s', 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': per_step * 1e3, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f32', 'data': 'synthetic', 'gpu_launches': 0,
        'config': {'workload': WORKLOAD, 'batch_per_gpu': 64, 'global_batch': 64 * args.gpus, 'parallelism': f'dp{args.gpus}', 'seed': SEED,
                   'cpu_sample': f'{sample} of the 64 samples of a step per timed forward'},
        'cpu_baseline': {'value': sps, 'unit': 'samples/s', 'cores': cores, 'kind': 'port',
                         'sample': f'{sample} samples per step (1/8 of the 64-sample batch), torch CPU fp32, {cores} threads'},
        'e2e': {'value': sps, 'unit': 'samples/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line), flush=True)


def micro_cases(device):
    """Single-op workloads at the benchmark's shapes: name -> (callable, algorithmic bytes, flops)."""
    from spgt_b200 import ops
    g = torch.Generator(device='cpu').manual_seed(2)
    rnd = lambda *shape: torch.randn(*shape, generator=g).to(device)
    cases = {}

    def attn(B=64, H=4, S=2809):
        Q, K, V = rnd(B, H, 34, S), rnd(B, H, 34, S), rnd(B, H, 34, S)
        return (lambda: ops.galerkin_attention(Q, K, V)), 4 * B * H * 34 * S * 4, 4 * B * H * 34 * 34 * S
    cases['attn'] = attn
    cases['attn_1849'] = lambda: attn(64, 4, 1849)

    def skinny(S):
        def make():
            A, Bm = rnd(64, 32, S), rnd(64, S, 32)
            ws = torch.empty(ops.skinny_gemm_workspace_bytes(32, 32, S, 64), dtype=torch.uint8, device=device)
            return (lambda: ops.batched_skinny_gemm(A, Bm, 1.0 / S, ws)), 64 * (2 * S * 32 + 32 * 32) * 4, 64 * 2 * S * 32 * 32
        return make
    for S in (1849, 19881, 44521):
        cases[f'skinny_{S}'] = skinny(S)

    def spectral(B=8, r=211, m=12):
        x, wr, br = rnd(B, r, r, 32), rnd(32, 32) / 6, rnd(32)
        f0, f1 = rnd(m, m, 32, 32, 2) / 1024, rnd(m, m, 32, 32, 2) / 1024
        ws = torch.empty(int(ops.lib.spgt_spectral_workspace_bytes(B, r, m, 32)), dtype=torch.uint8, device=device)
        flops = B * r * (2 * 32 * 2 * m * r * 2 + 2 * r * 32 * 32) + B * 8 * 2 * m * r * m * 32 * 2
        return (lambda: ops.spectral_conv2d(x, wr, br, f0, f1, m, 'silu', ws)), 2 * B * r * r * 32 * 4 + 2 * 2 * m * m * 32 * 32 * 8, flops
    cases['spectral'] = spectral
    cases['spectral_b64'] = lambda: spectral(64)

    def qkv(B=64, S=2809):
        x, pos = rnd(B, S, 128), rnd(B, S, 2)
        w, b_, lw, lb = [rnd(128, 128) / 11 for _ in range(3)], [rnd(128) for _ in range(3)], rnd(4, 32), rnd(4, 32)
        fn = lambda: ops.projpos_qkv(x, w[0], b_[0], w[1], b_[1], w[2], b_[2], lw, lb, lw, lb, 1e-6, pos, 4, 32, 2)
        return fn, B * S * (128 + 2 + 3 * 136) * 4, 3 * 2 * B * S * 128 * 128
    cases['qkv'] = qkv

    def ffn(B=64, S=2809):
        x, w1, b1, w2, b2 = rnd(B * S, 128), rnd(128, 256) / 11, rnd(256), rnd(256, 128) / 16, rnd(128)
        def fn():
            h = ops.linear(x, w1, b1, 256, 'relu')
            return ops.linear(h, w2, b2, 128, None, x)
        return fn, B * S * (128 + 256 + 256 + 128 + 128) * 4, 2 * 2 * B * S * 128 * 256
    cases['ffn'] = ffn

    def conv(B=64, Hh=106, C=128):
        x, w, b_ = rnd(B, Hh, Hh, C), rnd(9 * C, C) / 34, rnd(C)
        y = torch.empty_like(x)
        return (lambda: ops.conv3x3(x, 0, C, w, b_, y, 0, C, 'silu2')), 2 * B * Hh * Hh * C * 4, 2 * B * Hh * Hh * 9 * C * C
    cases['conv128'] = conv

    def ffn_tc(B=64, S=2809):
        x, w1, b1, w2, b2 = rnd(B * S, 128), ops.TcWeight(rnd(128, 256) / 11), rnd(256), ops.TcWeight(rnd(256, 128) / 16), rnd(128)
        def fn():
            h = ops.linear_tc(x, w1, b1, 'relu')
            return ops.linear_tc(h, w2, b2, None, x)
        return fn, B * S * (128 + 256 + 256 + 128 + 128) * 4, 2 * 2 * B * S * 128 * 256
    cases['ffn_tc'] = ffn_tc

    def ffn_fused(B=64, S=2809):
        x, w1, b1, w2, b2 = rnd(B * S, 128), ops.TcWeight(rnd(128, 256) / 11), rnd(256), ops.TcWeight(rnd(256, 128) / 16), rnd(128)
        return (lambda: ops.ffn_tc(x, w1, b1, w2, b2, 'relu', x)), B * S * (128 + 128 + 128) * 4, 2 * 2 * B * S * 128 * 256
    cases['ffn_fused'] = ffn_fused

    def lin_tc(B=64, S=2809, K=128, N=128, res=False):
        x, w, b_ = rnd(B * S, K), ops.TcWeight(rnd(K, N) / 11), rnd(N)
        r = rnd(B * S, N) if res else None
        return (lambda: ops.linear_tc(x, w, b_, None, r)), B * S * (K + N + (N if res else 0)) * 4, 2 * B * S * K * N
    cases['lin_tc'] = lin_tc
    cases['lin_tc_k136'] = lambda: lin_tc(K=136, res=True)      # attention output projection + residual
    cases['lin_tc_res'] = lambda: lin_tc(res=True)
    cases['lin_tc_k136_nores'] = lambda: lin_tc(K=136)
    cases['lin_tc_k160'] = lambda: lin_tc(K=160)
    cases['lin_tc_k256'] = lambda: lin_tc(K=256)
    cases['lin_tc_n32'] = lambda: lin_tc(N=32)

    def qkv_tc(B=64, S=2809):
        x, pos = rnd(B, S, 128), rnd(B, S, 2)
        w, b_, lw, lb = ops.TcWeight(rnd(128, 384) / 11), [rnd(128) for _ in range(3)], rnd(4, 32), rnd(4, 32)
        fn = lambda: ops.projpos_qkv_tc(x, w, b_[0], b_[1], b_[2], lw, lb, lw, lb, 1e-6, pos, 4, 32, 2)
        return fn, B * S * (128 + 2 + 3 * 136) * 4, 3 * 2 * B * S * 128 * 128
    cases['qkv_tc'] = qkv_tc

    def conv_tc(B=64, Hh=106, C=128):
        x, w, b_ = rnd(B, Hh, Hh, C), ops.TcWeight(rnd(9 * C, C) / 34), rnd(C)
        y = torch.empty_like(x)
        return (lambda: ops.conv3x3_tc(x, 0, C, w, b_, y, 0, C, 'silu2')), 2 * B * Hh * Hh * C * 4, 2 * B * Hh * Hh * 9 * C * C
    cases['conv128_tc'] = conv_tc

    def head_tc(B=64, r=211):
        x, w1, b1, w2 = rnd(B, r, r, 32), ops.TcWeight(rnd(32, 128) / 6), rnd(128), rnd(128)
        return (lambda: ops.decoder_head_tc(x, w1, b1, w2, 0.1, 1.0, 0.0, True, 'silu')), B * r * r * 33 * 4, 2 * B * r * r * 32 * 128
    cases['head_tc'] = head_tc

    def darcy_cg(B=16, K=421, iters=200):
        # `iters` conjugate-gradient iterations of the batched finite-volume Darcy solve (data generator), float64:
        # per iteration and node 13 array accesses of 8 bytes (step A: z, p, a in, p, q out; step B: a, p, q, x, r in, x, r, z out)
        a = torch.where(torch.randn(B, K, K, device=device) >= 0, 12.0, 3.0).double()
        f = torch.ones(B, K, K, device=device, dtype=torch.float64)
        p = torch.empty_like(a)
        ws = torch.empty(int(ops.lib.spgt_darcy_fv_workspace_bytes(B, K)), dtype=torch.uint8, device=device)

        def fn():
            code = ops.lib.spgt_darcy_fv_solve(a.data_ptr(), f.data_ptr(), p.data_ptr(), B, K, iters, 1e-300, iters, ws.data_ptr(),
                                               ws.numel(), None, None, torch.cuda.current_stream().cuda_stream)
            assert code == -7, code                     # stops at the iteration limit by construction
        return fn, 13 * 8 * B * K * K * iters, 20 * B * K * K * iters
    cases['darcy_cg'] = darcy_cg
    return cases


def run_micro(args):
    """One op in isolation: JSON line with achieved GB/s (algorithmic bytes) and TFLOP/s; L2 is flushed between
    timed launches by writing a 256 MB buffer."""
    from spgt_b200 import ops
    device = torch.device('cuda', 0)
    torch.cuda.set_device(device)
    fn, nbytes, flops = micro_cases(device)[args.micro]()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for _ in range(max(args.warmup, 1)):
        fn()
    times = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    med = times[len(times) // 2]
    peak, kind = measured_peak()
    print(json.dumps({'micro': args.micro, 'median_ms': med, 'min_ms': times[0], 'algorithmic_bytes': nbytes, 'flops': flops,
                      'GBps': nbytes / med / 1e6, 'frac_of_hbm_peak': nbytes / med / 1e6 / peak, 'peak_kind': kind,
                      'TFLOPs': flops / med / 1e9, 'steps': args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--micro', default=None, help='time one op in isolation (see micro_cases) instead of the model')
    ap.add_argument('--tune', default=None, help='key=value passed to spgt_set_tuning before running (experiments)')
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='spgt_b200', choices=['spgt_b200', 'reference'])
    ap.add_argument('--batch', type=int, default=64, help='samples per GPU per step')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-graphs', action='store_true', help='end-to-end leg launches the kernels eagerly instead of replaying CUDA graphs')
    ap.add_argument('--breakdown', action='store_true', help='also print a per-entry-point time table to stderr')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != 'reference' else args.warmup
    rank, world, local = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))

    if args.impl == 'reference':
        run_reference(args, rank)
        return
    if args.tune:
        from spgt_b200._lib import lib
        k, v = args.tune.split('=')
        assert lib.spgt_set_tuning(k.encode(), int(v)) == 0, 'unknown tuning key or value'
    if args.micro:
        run_micro(args)
        return

    from spgt_b200 import ops
    from spgt_b200.config.config_accessor import get_darcy_config
    from spgt_b200.dataset.darcy_dataset import GaussNormalizer, synthetic_darcy_batch
    from spgt_b200.engine.darcy_engine import HostInference
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D

    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group('nccl', init_method='env://', device_id=device)

    cfg = get_darcy_config(SUB_NODE, SUB_ATTN, num_frequence_mode=MODES)
    cfg['target_normalizer'] = GaussNormalizer()
    torch.manual_seed(SEED)
    model = Sp_GalerkinTransformer2D(cfg).to(device).eval()
    B = args.batch
    host = synthetic_darcy_batch(range(rank * B, (rank + 1) * B), FINE, SUB_NODE, SUB_ATTN, SEED)
    host = {k: v.pin_memory() for k, v in host.items() if k != 'coeff'}
    dev = {k: v.to(device) for k, v in host.items()}
    S, H, DPK = cfg['r_attn'] ** 2, cfg['num_head'], 34

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---------------- device-resident throughput ----------------
    for _ in range(args.warmup):
        model(dev['node'], dev['position'], dev['grid'])
    barrier()
    launches0 = ops.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks, ops.profile_ops(only=['spgt_galerkin_attn_fwd']) as prof:
        e0.record()
        for _ in range(args.steps):
            out = model(dev['node'], dev['position'], dev['grid'])
        e1.record()
        barrier()
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = ops.LAUNCHES - launches0
    attn_ms = prof.times_ms().get('spgt_galerkin_attn_fwd', [])
    attn_avg_ms = sum(attn_ms) / max(1, len(attn_ms))
    value = world * B * args.steps / (elapsed_ms * 1e-3)

    # ---------------- end to end through the host-facing API ----------------
    engine = HostInference(model, device, use_graphs=not args.no_graphs)
    outs = [torch.empty(B, cfg['r_node'], cfg['r_node'], 1, dtype=torch.float32, pin_memory=True) for _ in range(2)]
    engine.run([host] * args.warmup, [outs[i & 1] for i in range(args.warmup)])
    barrier()
    t0 = time.perf_counter()
    engine.run([host] * args.steps, [outs[i & 1] for i in range(args.steps)])
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    nbytes = engine.bytes_per_batch(host)
    e2e_value = world * B * args.steps / e2e_s

    # ---------------- roofline of the attention kernel ----------------
    peak, peak_kind = measured_peak()
    algo_bytes = 4 * B * H * DPK * S * 4                      # read Q, K, V and write out, fp32
    achieved = algo_bytes / (attn_avg_ms * 1e-3) / 1e9 if attn_avg_ms > 0 else None
    roofline = {'kernel': 'galerkin_attn_tc_kernel', 'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'peak_kind': peak_kind,
                'unit': 'GB/s', 'frac': (achieved / peak) if achieved else None, 'traffic': ATTN_TRAFFIC_BYTES,
                'algorithmic_bytes': algo_bytes, 'avg_launch_ms': attn_avg_ms, 'launches_timed': len(attn_ms)}

    if args.breakdown and rank == 0:
        with ops.profile_ops() as pall:
            model(dev['node'], dev['position'], dev['grid'])
        tm = pall.times_ms()
        tot = sum(sum(v) for v in tm.values())
        for k, v in sorted(tm.items(), key=lambda kv: -sum(kv[1])):
            print(f'{k:34s} calls {len(v):3d}  total {sum(v):8.3f} ms  {100 * sum(v) / tot:5.1f} %', file=sys.stderr)
            if len(v) > 1:
                print('    per call (us): ' + ' '.join(f'{1e3 * t:.0f}' for t in v), file=sys.stderr)
        print(f'{"sum":34s} {tot:8.3f} ms', file=sys.stderr)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = use_all_host_threads()
        sps, per_step = time_oracle(8, 3, 1)
        cpu = {'value': sps, 'unit': 'samples/s', 'cores': cores, 'kind': 'port',
               'sample': f'8 samples per forward (1/8 of the batch), 3 timed forwards after 1 warm-up, torch CPU fp32, {cores} threads'}

    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': 'samples/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': elapsed_ms / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'f32', 'data': 'synthetic',
            'config': {'workload': WORKLOAD, 'batch_per_gpu': B, 'global_batch': B * world, 'parallelism': f'dp{world}', 'seed': SEED,
                       'l2_policy': 'per-step working set (several GB of activations) is far larger than the 126 MB L2'},
            'clocks': clocks.summary(), 'gpu_launches': launches,
            'e2e': {'value': e2e_value, 'unit': 'samples/s', 'h2d_bytes_per_step': nbytes['h2d'], 'd2h_bytes_per_step': nbytes['d2h'],
                    'ms_per_step': e2e_s * 1e3 / args.steps},
            'roofline': roofline, 'cpu_baseline': cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
