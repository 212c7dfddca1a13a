"""Timing sweeps over resolution and batch, after the reference's evaluate/sp_galerkin.py, evaluate/sp_fno2d.py and
evaluate/sp_darcy_breakdown.py: each op of this library ("Exts") next to the plain PyTorch formulation the reference
calls "Orig" (torch.matmul / nn.functional on the same GPU, TF32 off), forward only; and the four components of the
whole model (down-scaler, encoder layers, up-scaler, spectral regressor) on the fused kernels next to the
reference-structure path (this library's attention / projection / data-movement ops, library ops for the rest).

    python -m spgt_b200.evaluate.sp_sweeps [skinny_resolution skinny_batch projpos attention fno2d breakdown ...]

Timing: CUDA events around each call after warm-up, median of `repeat` calls, a 256 MB buffer written between calls so
that no call finds its inputs in L2.  Output: one markdown table per sweep on stdout.
"""
import math
import sys
from typing import Callable, Dict, List

import torch

from .. import ops
from ..network.sp_layer import Sp_SpectralConv2D


def _time(fn: Callable[[], object], repeat: int = 10, warmup: int = 3) -> float:
    flush = _time.flush
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(repeat):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def _table(title: str, key: str, rows: List[Dict]) -> None:
    print(f'\n### {title}\n')
    print(f'| {key} | Orig (torch) ms | Exts (spgt_b200) ms | speed-up |')
    print('|---:|---:|---:|---:|')
    for r in rows:
        print(f"| {r['key']} | {r['orig']:.4f} | {r['exts']:.4f} | {r['orig'] / r['exts']:.2f}x |")
    sys.stdout.flush()


def time_skinny_gemm_wrt_resolution(resolution_list=(32, 64, 128, 256, 512), batch=16, d_posk=32):
    rows = []
    for r in resolution_list:
        S = r * r
        A, B = torch.rand(batch, d_posk, S, device='cuda'), torch.rand(batch, S, d_posk, device='cuda')
        ws = torch.empty(ops.skinny_gemm_workspace_bytes(d_posk, d_posk, S, batch), dtype=torch.uint8, device='cuda')
        rows.append(dict(key=r, orig=_time(lambda: torch.matmul(A, B)), exts=_time(lambda: ops.batched_skinny_gemm(A, B, 1.0, ws))))
    _table(f'skinny GEMM [batch {batch}, {d_posk} x S] x [S x {d_posk}], S = resolution^2', 'resolution', rows)


def time_skinny_gemm_wrt_batch(batch_list=(4, 8, 16, 32, 64, 128, 256), resolution=256, d_posk=32):
    rows, S = [], resolution * resolution
    for b in batch_list:
        A, B = torch.rand(b, d_posk, S, device='cuda'), torch.rand(b, S, d_posk, device='cuda')
        ws = torch.empty(ops.skinny_gemm_workspace_bytes(d_posk, d_posk, S, b), dtype=torch.uint8, device='cuda')
        rows.append(dict(key=b, orig=_time(lambda: torch.matmul(A, B)), exts=_time(lambda: ops.batched_skinny_gemm(A, B, 1.0, ws))))
    _table(f'skinny GEMM, resolution {resolution} (S = {S}), {d_posk} x S x {d_posk}', 'batch', rows)


def _projpos_lnorm_torch(x, w, b, lnw, lnb, pos, eps, H, d):
    B, S, _ = x.shape
    h = (x @ w + b).view(B, S, H, d)
    h = torch.nn.functional.layer_norm(h, (d,), None, None, eps) * lnw + lnb
    p = pos.view(B, S, 1, -1).expand(B, S, H, pos.shape[-1])
    return torch.cat([p, h], dim=-1).permute(0, 2, 3, 1).contiguous()


def time_projpos_lnorm_wrt_resolution(resolution_list=(32, 64, 128, 256), batch=16, num_head=4, dim_head=32, dim_position=2, eps=1e-5):
    rows, D = [], num_head * dim_head
    for r in resolution_list:
        S = r * r
        x, w, b = torch.rand(batch, S, D, device='cuda'), torch.rand(D, D, device='cuda') / D, torch.rand(D, device='cuda')
        lnw, lnb = torch.rand(num_head, dim_head, device='cuda'), torch.rand(num_head, dim_head, device='cuda')
        pos = torch.rand(batch, S, dim_position, device='cuda')
        rows.append(dict(key=r, orig=_time(lambda: _projpos_lnorm_torch(x, w, b, lnw, lnb, pos, eps, num_head, dim_head)),
                         exts=_time(lambda: ops.projpos_lnorm(x, w, b, lnw, lnb, pos, eps, num_head, dim_head, dim_position))))
    _table(f'projection + per-head LayerNorm + position rows, batch {batch}, D = {D}', 'resolution', rows)


def time_attention_wrt_resolution(resolution_list=(32, 53, 64, 106, 128, 256), batch=16, num_head=4, d_posk=34):
    rows = []
    for r in resolution_list:
        S = r * r
        Q, K, V = (torch.rand(batch, num_head, d_posk, S, device='cuda') for _ in range(3))
        orig = lambda: torch.matmul(Q.transpose(-2, -1), torch.matmul(K, V.transpose(-2, -1)) / S)
        rows.append(dict(key=r, orig=_time(orig), exts=_time(lambda: ops.galerkin_attention(Q, K, V))))
    _table(f'Galerkin attention Q^T (K V^T / S), batch {batch}, {num_head} heads, d_posk {d_posk}', 'resolution', rows)


def _spectral_torch(x, wr, br, fw0, fw1, m):
    B, r, _, C = x.shape
    res = x @ wr + br
    xf = torch.fft.rfft2(x.permute(0, 3, 1, 2), s=(r, r), norm='ortho')
    out = torch.zeros(B, C, r, r // 2 + 1, dtype=torch.cfloat, device=x.device)
    w0, w1 = torch.view_as_complex(fw0), torch.view_as_complex(fw1)          # [m, m, in, out]
    out[:, :, :m, :m] = torch.einsum('bixy,xyio->boxy', xf[:, :, :m, :m], w0)
    out[:, :, -m:, :m] = torch.einsum('bixy,xyio->boxy', xf[:, :, -m:, :m], w1)
    y = torch.fft.irfft2(out, s=(r, r), norm='ortho').permute(0, 2, 3, 1)
    return torch.nn.functional.silu(y + res)


def time_fno2d_wrt_resolution(resolution_list=(32, 64, 128, 211, 256), batch=4, width=32):
    rows = []
    for r in resolution_list:
        m = min(16, math.ceil(math.sqrt(r)))
        layer = Sp_SpectralConv2D(width, width, m, 0.0, 'silu').cuda()
        x = torch.rand(batch, r, r, width, device='cuda')
        wr, br = layer.residual_layer.weight.detach().t().contiguous(), layer.residual_layer.bias.detach()
        fw0, fw1 = (p.detach().contiguous() for p in layer.fourier_weight)
        with torch.no_grad():
            rows.append(dict(key=f'{r} (m={m})', orig=_time(lambda: _spectral_torch(x, wr, br, fw0, fw1, m)), exts=_time(lambda: layer(x))))
    _table(f'spectral layer (FNO2d block), batch {batch}, width {width}', 'resolution', rows)


def time_model_breakdown_wrt_resolution(resolution_list=(128, 211, 256, 64), batch=4):
    """Forward time of the model's four components at fine grid R x R (every node kept) and attention grid R/2, as the
    reference's breakdown sweep sets them up (evaluate/sp_darcy_breakdown.py:21-40); Fourier modes ceil(sqrt(R)) capped at
    the 16 the fused spectral kernels take.  "Orig" = the reference-structure path, "Exts" = the fused kernels."""
    from ..config.config_accessor import get_darcy_config
    from ..dataset.darcy_dataset import GaussNormalizer
    from ..network.sp_model import Sp_GalerkinTransformer2D
    for R in resolution_list:
        modes = min(16, math.ceil(math.sqrt(R)))
        cfg = get_darcy_config(1, 2, num_frequence_mode=modes, clamp_attn=False, fine_resolution=R)
        cfg['target_normalizer'] = GaussNormalizer()
        torch.manual_seed(R)
        model = Sp_GalerkinTransformer2D(cfg).cuda().eval()
        r, ra = cfg['r_node'], cfg['r_attn']
        node, grid = torch.rand(batch, r, r, 1, device='cuda'), torch.rand(batch, r, r, 2, device='cuda')
        pos = torch.rand(batch, ra, ra, 2, device='cuda')
        rows = []
        with torch.no_grad():
            xd = model.down_scaler(node)
            xe = model.encoder_mixer(xd, pos)
            xu = model.up_scaler(xe)
            rows.append(dict(key='down-scaler', orig=_time(lambda: model.down_scaler.forward_train(node)), exts=_time(lambda: model.down_scaler(node))))
            rows.append(dict(key=f'{len(model.encoder_mixer.layers)} encoder layers', orig=_time(lambda: model.encoder_mixer.forward_train(xd, pos)),
                             exts=_time(lambda: model.encoder_mixer(xd, pos))))
            rows.append(dict(key='up-scaler', orig=_time(lambda: model.up_scaler.forward_train(xe)), exts=_time(lambda: model.up_scaler(xe))))
            rows.append(dict(key='spectral regressor', orig=_time(lambda: model.decoder_regressor.forward_train(xu, grid)),
                             exts=_time(lambda: model.decoder_regressor(xu, grid))))
            rows.append(dict(key='whole model', orig=_time(lambda: model.forward_train(node, pos, grid)), exts=_time(lambda: model(node, pos, grid))))
        _table(f'model components, fine grid {r} x {r}, attention grid {ra} x {ra}, {modes} modes, batch {batch}', 'component', rows)


SWEEPS = {'skinny_resolution': time_skinny_gemm_wrt_resolution, 'skinny_batch': time_skinny_gemm_wrt_batch,
          'projpos': time_projpos_lnorm_wrt_resolution, 'attention': time_attention_wrt_resolution, 'fno2d': time_fno2d_wrt_resolution,
          'breakdown': time_model_breakdown_wrt_resolution}


def main(argv):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    _time.flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda')
    print(f'# Op sweeps on {torch.cuda.get_device_name(0)} (fp32; "Orig" = PyTorch ops with TF32 off, "Exts" = this library)')
    for name in (argv or list(SWEEPS)):
        SWEEPS[name]()


if __name__ == '__main__':
    main(sys.argv[1:])
