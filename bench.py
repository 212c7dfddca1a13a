#!/usr/bin/env python
"""Darcy Galerkin Transformer inference benchmark (211 x 211 fine grid, 53 x 53 attention grid, global batch 64).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One rank per GPU (torchrun for N > 1).  A step is one forward of the full model over the GLOBAL batch of 64 synthetic
Darcy coefficient fields, sharded 64/N per rank (strong scaling, no collective inside the forward); rank 0 prints one
JSON line.
  value         samples/s with the inputs resident in HBM: blocks of K replays of the captured forward, CUDA events, max
                over ranks per block, median block.
  e2e           the same metric through the host-facing API: per step every rank uploads its slice from pinned host
                memory, runs the forward, all ranks all-gather the predictions and all-reduce the validation metric
                (NCCL), rank 0 downloads the gathered predictions; uploads / downloads overlap the next / previous step.
  roofline      the Galerkin attention kernel: CUDA events around each of its launches in a separate eagerly launched
                pass over the same inputs; roofline_spectral the same for the spectral layer's launches.
  cpu_baseline  the reference's own CPU model (or, where its files are not staged, the CPU restatement) on a bounded sample.
`--impl reference` times that CPU path alone, with all host threads, on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
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
GLOBAL_BATCH = 64
CPU_SAMPLE = 8                     # samples per forward of the CPU legs (a bounded sample of the 64-sample step)
# DRAM bytes (read + write) of one launch at batch 64 from the committed ncu summaries of these kernels; they grow in
# proportion to the batch, so a rank that holds 64/N samples is charged 1/N of them.
ATTN_TRAFFIC_BYTES_B64 = 343_600_000
SPECTRAL_TRAFFIC_BYTES_B64 = 1_174_600_000


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


WORKLOAD = ('full Darcy Galerkin Transformer forward, fine grid 211x211, attention grid 53x53, 6 encoder '
            'layers (hidden 128, 4 heads, FFN 256), FNO2d regressor (2 spectral layers, width 32, 12 modes)')


def random_state(seed: int = SEED, modes: int = MODES):
    """Random-init weights of the benchmark architecture, keyed and laid out as the reference's Sp_GalerkinTransformer2D
    state_dict (network/sp_model.py:67-89) and drawn with the reference's initialisers: torch's Linear / Conv2d defaults,
    xavier_uniform(gain 0.01) + 0.01 I for the Q/K/V matrices with zero biases and unit LayerNorm (network/sp_layer.py:39-50),
    xavier_normal with gain sqrt(in + out) / (in * out) for the Fourier weights (network/sp_layer.py:119-123).  Plain
    torch, no package import: both arms of the benchmark build their weights from this one function."""
    g = torch.Generator().manual_seed(seed)
    st = {}

    def dense(prefix, out_f, fan_in, shape):
        bound = 1.0 / math.sqrt(fan_in)
        st[prefix + '.weight'] = (torch.rand(*shape, generator=g) * 2 - 1) * bound
        st[prefix + '.bias'] = (torch.rand(out_f, generator=g) * 2 - 1) * bound

    for i, (co, ci) in enumerate(((128, 1), (42, 128), (42, 42), (44, 42))):
        dense(f'down_scaler.conv{i}.conv_layer', co, ci * 9, (co, ci, 3, 3))
    for l in range(6):
        a = f'encoder_mixer.layers.{l}.attention_layer.'
        for n in 'QKV':
            st[a + 'weight_' + n] = torch.nn.init.xavier_uniform_(torch.empty(128, 128), gain=0.01, generator=g) + 0.01 * torch.eye(128)
            st[a + 'bias_' + n] = torch.zeros(128)
        for n in 'KV':
            st[a + 'ln_weight_' + n], st[a + 'ln_bias_' + n] = torch.ones(4, 32), torch.zeros(4, 32)
        dense(a + 'fc_layer', 128, 136, (128, 136))
        f = f'encoder_mixer.layers.{l}.ffn_layer.'
        dense(f + 'layer1', 256, 128, (256, 128))
        dense(f + 'layer2', 128, 256, (128, 256))
    dense('up_scaler.conv.conv_layer', 128, 128 * 9, (128, 128, 3, 3))
    d = 'decoder_regressor.'
    dense(d + 'spatial_fc_layer', 32, 130, (32, 130))
    for l in range(2):
        dense(d + f'layers.{l}.residual_layer', 32, 32, (32, 32))
        for k in range(2):
            st[d + f'layers.{l}.fourier_weight.{k}'] = torch.nn.init.xavier_normal_(
                torch.empty(modes, modes, 32, 32, 2), gain=math.sqrt(64.0) / 1024.0, generator=g)
    dense(d + 'ffn_layer.layer1', 128, 32, (128, 32))
    dense(d + 'ffn_layer.layer2', 1, 128, (1, 128))
    return st


def use_all_host_threads() -> int:
    """The launcher of multi-rank runs exports OMP_NUM_THREADS=1; the CPU legs use every core this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def time_cpu_path(steps: int, warmup: int):
    """The reference's CPU model (oracle/_ref, staged by oracle/build_ref.py) or, without it, the CPU restatement, on
    CPU_SAMPLE of the benchmark's samples per forward.  Returns (samples/s, s per forward, kind, cores)."""
    from oracle import gt_oracle as O
    from oracle import ref_runner as R
    cores = use_all_host_threads()
    ocfg = O.default_config(FINE, SUB_NODE, SUB_ATTN, MODES)
    data = R.synthetic_batch(range(CPU_SAMPLE), FINE, SUB_NODE, SUB_ATTN, SEED)
    fwd, kind = R.make_forward(ocfg, random_state())
    for _ in range(warmup):
        fwd(data['node'], data['position'], data['grid'])
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fwd(data['node'], data['position'], data['grid'])
        times.append(time.perf_counter() - t0)
    per = sum(times) / len(times)
    return CPU_SAMPLE / per, per, kind, cores


def run_reference(args, rank):
    """--impl reference: the CPU path alone on rank 0 (other ranks have nothing to do and return at once)."""
    if rank != 0:
        return
    sps, per_step, kind, cores = time_cpu_path(args.steps, args.warmup)
    sample = (f'{CPU_SAMPLE} of the {GLOBAL_BATCH} samples of a step per timed forward, '
              + ("the reference's GalerkinTransformer2D (network/model.py)" if kind == 'reference' else 'CPU restatement of the reference model')
              + f', torch CPU fp32, {cores} threads')
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': sps, 'unit': 'samples/s', 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': per_step * 1e3, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': 'f32', 'data': 'synthetic', 'gpu_launches': 0,
        'config': {'workload': WORKLOAD, 'global_batch': GLOBAL_BATCH, 'batch_per_gpu': GLOBAL_BATCH // max(1, args.gpus),
                   'parallelism': f'dp{args.gpus}', 'seed': SEED, 'cpu_sample': sample},
        'cpu_baseline': {'value': sps, 'unit': 'samples/s', 'cores': cores, 'kind': kind, 'sample': sample},
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

    def spectral(B=8, r=211, m=12, act='silu'):
        x, wr, br = rnd(B, r, r, 32), rnd(32, 32) / 6, rnd(32)
        f0, f1 = rnd(m, m, 32, 32, 2) / 1024, rnd(m, m, 32, 32, 2) / 1024
        ws = torch.empty(int(ops.lib.spgt_spectral_workspace_bytes(B, r, m, 32)), dtype=torch.uint8, device=device)
        flops = B * r * (2 * 32 * 2 * m * r * 2 + 2 * r * 32 * 32) + B * 8 * 2 * m * r * m * 32 * 2
        return (lambda: ops.spectral_conv2d(x, wr, br, f0, f1, m, act, ws)), 2 * B * r * r * 32 * 4 + 2 * 2 * m * m * 32 * 32 * 8, flops
    cases['spectral'] = spectral
    cases['spectral_b64'] = lambda: spectral(64)
    cases['spectral_b64_relu'] = lambda: spectral(64, act='relu')

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

    def conv_tc_down(B=64, Hh=106, Cin=44, Cout=44):
        # down-scaler shapes: 42 / 44 channels zero-padded to 44 (64-wide column tile)
        x, w, b_ = rnd(B, Hh, Hh, Cin), ops.TcWeight(rnd(9 * Cin, Cout) / 20), rnd(Cout)
        y = torch.empty(B, Hh, Hh, Cout, device=device)
        return (lambda: ops.conv3x3_tc(x, 0, Cin, w, b_, y, 0, Cout, 'silu')), B * Hh * Hh * (Cin + Cout) * 4, 2 * B * Hh * Hh * 9 * Cin * Cout
    cases['conv44_tc'] = conv_tc_down
    cases['conv128to44_tc'] = lambda: conv_tc_down(Cin=128)

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
    ap.add_argument('--batch', type=int, default=GLOBAL_BATCH, help='global batch per step, sharded evenly over the ranks')
    ap.add_argument('--min-seconds', type=float, default=1.0, help='repeat the K-step block until this much time has been measured')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--e2e-download', default='metric', choices=['metric', 'predictions'],
                    help="what the end-to-end leg reads back per step: the reduced metric (as the reference's driver does) or also the gathered predictions")
    ap.add_argument('--no-graphs', action='store_true', help='launch the kernels eagerly instead of replaying CUDA graphs')
    ap.add_argument('--no-weak-leg', action='store_true', help='skip the secondary 64-samples-per-GPU measurement of multi-GPU runs')
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
    from spgt_b200.engine.darcy_engine import GraphedForward, HostInference
    from spgt_b200.network.sp_model import Sp_GalerkinTransformer2D
    from spgt_b200.run.ddp_darcy_inference import ShardedGather, shard_range

    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group('nccl', init_method='env://', device_id=device)
    if args.batch % world != 0:
        raise SystemExit(f'--batch {args.batch} does not split evenly over {world} ranks')

    cfg = get_darcy_config(SUB_NODE, SUB_ATTN, num_frequence_mode=MODES)
    cfg['target_normalizer'] = GaussNormalizer()
    model = Sp_GalerkinTransformer2D(cfg)
    model.load_state_dict(random_state(), strict=True)
    model = model.to(device).eval()
    G = args.batch
    begin, end = shard_range(G, rank, world)
    B = end - begin                                           # samples of this rank per step
    r, S, H, DPK = cfg['r_node'], cfg['r_attn'] ** 2, cfg['num_head'], 34

    def make_host(indices):
        h = synthetic_darcy_batch(indices, FINE, SUB_NODE, SUB_ATTN, SEED)
        h['target'] = h.pop('coeff') * 0.01                  # stands in for the PDE solution the validation metric compares with
        return {k: v.pin_memory() for k, v in h.items()}
    host = make_host(range(begin, end))
    dev = {k: v.to(device) for k, v in host.items()}

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

    def timed_blocks(step_fn, steps, min_seconds):
        """Blocks of exactly `steps` calls, each bracketed by barrier + synchronize and timed with CUDA events on the
        launching stream, max over ranks; repeated until min_seconds have been measured.  Returns the block times (ms)."""
        blocks, total = [], 0.0
        while True:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step_fn()
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1))
            blocks.append(ms)
            total += ms
            if (total >= min_seconds * 1e3 and len(blocks) >= 3) or len(blocks) >= 200:
                return blocks

    def device_leg(inputs, steps, min_seconds):
        if args.no_graphs:
            fwd = lambda: model(inputs['node'], inputs['position'], inputs['grid'])
        else:
            graphed = GraphedForward(model, inputs['node'], inputs['position'], inputs['grid'], own_inputs=False)
            fwd = lambda: graphed(inputs['node'], inputs['position'], inputs['grid'])
        for _ in range(args.warmup):
            fwd()
        return timed_blocks(fwd, steps, min_seconds)

    # ---------------- kernels per forward (counted on an eager pass) ----------------
    for _ in range(2):
        model(dev['node'], dev['position'], dev['grid'])     # weight images, tables and kernel attributes are set up here
    l0 = ops.LAUNCHES
    model(dev['node'], dev['position'], dev['grid'])
    launches_per_forward = ops.LAUNCHES - l0

    # ---------------- device-resident throughput ----------------
    with ClockSampler(local) as clocks:
        blocks = device_leg(dev, args.steps, args.min_seconds)
    blocks_sorted = sorted(blocks)
    elapsed_ms = blocks_sorted[len(blocks_sorted) // 2]
    value = G * args.steps / (elapsed_ms * 1e-3)

    # ---------------- end to end through the host-facing API ----------------
    # Every step uploads that step's samples (the coefficient field `node`); the node coordinates (`position`, `grid`) and the
    # synthetic stand-in for the solution the metric compares with are the same host tensors in every step and are
    # uploaded once per staging slot.
    engine = HostInference(model, device, use_graphs=not args.no_graphs, static_keys=('position', 'grid', 'target'))
    gather = ShardedGather(G, rank, world, (r, r, 1), device, download=args.e2e_download)
    engine.run([host] * args.warmup, post=gather)
    barrier()
    t0 = time.perf_counter()
    results = engine.run([host] * args.steps, post=gather)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    nb = engine.bytes_per_batch(host)
    e2e_value = G * args.steps / e2e_s
    metric_value = gather.metric(args.steps - 1)

    # ---------------- the gathered predictions, checked after the timed region ----------------
    gather_check = None
    pred_local = model(dev['node'], dev['position'], dev['grid'])
    csum = pred_local.double().sum().reshape(1)
    if world > 1:
        sums = torch.empty(world, dtype=torch.float64, device=device)
        dist.all_gather_into_tensor(sums, csum)
    else:
        sums = csum
    if rank == 0:
        # the last step's gathered predictions: their pinned host copy, or (metric-only download) fetched from the device now
        full = results[-1] if args.e2e_download == 'predictions' else gather.last_full.cpu()
        ok = torch.equal(full[begin:end], pred_local.cpu())
        for rk in range(world):
            b, e = shard_range(G, rk, world)
            ok = ok and abs(float(full[b:e].double().sum()) - float(sums[rk])) <= 1e-9 * abs(float(sums[rk]))   # rank rk's block sits where the global order puts it
        gather_check = 'ok' if ok else 'MISMATCH'

    # ---------------- rooflines of the attention kernel and the spectral layer (separate eager pass) ----------------
    names = ['spgt_galerkin_attn_fwd', 'spgt_spectral_conv2d_fwd']
    with ops.profile_ops(only=names) as prof:
        for _ in range(args.steps):
            model(dev['node'], dev['position'], dev['grid'])
    tm = prof.times_ms()
    peak, peak_kind = measured_peak()

    def roofline(name, kernel, algo_bytes, traffic_b64):
        t = tm.get(name, [])
        avg = sum(t) / max(1, len(t))
        achieved = algo_bytes / (avg * 1e-3) / 1e9 if avg > 0 else None
        return {'kernel': kernel, 'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'peak_kind': peak_kind, 'unit': 'GB/s',
                'frac': (achieved / peak) if achieved else None,
                'traffic': (traffic_b64 * B // 64) if traffic_b64 else None, 'algorithmic_bytes': algo_bytes,
                'avg_launch_ms': avg, 'launches_timed': len(t)}
    roof_attn = roofline('spgt_galerkin_attn_fwd', 'galerkin_attn_tc_kernel', 4 * B * H * DPK * S * 4, ATTN_TRAFFIC_BYTES_B64)
    # spectral layer: read x once, write y once (fp32, 32 channels) + the complex mode weights; one entry-point call = all its kernels
    roof_spec = roofline('spgt_spectral_conv2d_fwd', 'spectral layer (all kernels of one call)',
                         2 * B * r * r * 32 * 4 + 2 * 2 * MODES * MODES * 32 * 32 * 8, SPECTRAL_TRAFFIC_BYTES_B64)

    # ---------------- secondary: fixed 64 samples per GPU (weak scaling) ----------------
    weak = None
    if world > 1 and not args.no_weak_leg:
        wdev = {k: v.to(device) for k, v in make_host(range(rank * 64, rank * 64 + 64)).items()}
        wb = sorted(device_leg(wdev, args.steps, 0.0))
        wms = wb[len(wb) // 2]
        weak = {'batch_per_gpu': 64, 'global_batch': 64 * world, 'value': world * 64 * args.steps / (wms * 1e-3), 'ms_per_step': wms / args.steps}
        del wdev

    if args.breakdown and rank == 0:
        with ops.profile_ops() as pall:
            model(dev['node'], dev['position'], dev['grid'])
        tb = pall.times_ms()
        tot = sum(sum(v) for v in tb.values())
        for k, v in sorted(tb.items(), key=lambda kv: -sum(kv[1])):
            print(f'{k:34s} calls {len(v):3d}  total {sum(v):8.3f} ms  {100 * sum(v) / tot:5.1f} %', file=sys.stderr)
            if len(v) > 1:
                print('    per call (us): ' + ' '.join(f'{1e3 * t:.0f}' for t in v), file=sys.stderr)
        print(f'{"sum":34s} {tot:8.3f} ms', file=sys.stderr)

    ops.check_tc_status('bench')                              # a kernel that gave up on a wait would have produced garbage timings

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sps, per_step, kind, cores = time_cpu_path(5, 1)
        cpu = {'value': sps, 'unit': 'samples/s', 'cores': cores, 'kind': kind,
               'sample': f'{CPU_SAMPLE} samples per forward (1/8 of the global batch), 5 timed forwards after 1 warm-up, torch CPU fp32, {cores} threads'}

    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': 'samples/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': elapsed_ms / args.steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
            'dtype': 'f32', 'data': 'synthetic',
            'config': {'workload': WORKLOAD, 'global_batch': G, 'batch_per_gpu': B, 'parallelism': f'dp{world}', 'seed': SEED,
                       'forward': 'eager launches' if args.no_graphs else 'CUDA graph replay',
                       'l2_policy': f'per-step working set ({B * 47} MB of activations per rank) is larger than the 126 MB L2',
                       'timing': f'median of {len(blocks)} blocks of {args.steps} steps (CUDA events, max over ranks per block)'},
            'clocks': clocks.summary(), 'gpu_launches': launches_per_forward * args.steps, 'launches_per_forward': launches_per_forward,
            'block_ms': {'min': blocks_sorted[0], 'median': elapsed_ms, 'max': blocks_sorted[-1], 'n': len(blocks)},
            'e2e': {'value': e2e_value, 'unit': 'samples/s', 'h2d_bytes_per_step': nb['h2d'] * world, 'd2h_bytes_per_step': (G * r * r * 4 + 16 * world) if args.e2e_download == 'predictions' else 32 * world,
                    'downloads': args.e2e_download,
                    'ms_per_step': e2e_s * 1e3 / args.steps,
                    'collectives_per_step': 0 if world == 1 else 2, 'gather_check': gather_check, 'metric': metric_value},
            'roofline': roof_attn, 'roofline_spectral': roof_spec, 'cpu_baseline': cpu, 'weak_64_per_gpu': weak,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
