"""Tensor-level wrappers of the C ABI: torch supplies device memory and the current stream, nothing else.

Every function checks device, dtype and contiguity (the kernels read raw pointers), allocates its output with
torch.empty on the input's device and launches on torch's current stream.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor

from ._lib import lib, check

ACT = {None: 0, 'none': 0, 'relu': 1, 'silu': 2, 'silu2': 3}


def act_code(name) -> int:
    """The reference selects SiLU for 'silu' and ReLU for any other string (network/layer.py:14,163)."""
    if name in ACT:
        return ACT[name]
    return 1


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# kernels launched by one call of each entry point (everything else launches one)
_KERNELS_PER_CALL = {'spgt_batched_skinny_gemm': 2, 'spgt_galerkin_attn_bwd': 2, 'spgt_projpos_bwd_elementwise': 2}
LAUNCHES = 0          # running count of kernels launched through this module
_PROFILE = None       # None, or a dict name -> list of (start_event, end_event) filled while profiling


def _call(name: str, *args, kernels: int = None) -> None:
    """`kernels`: how many kernels this call launches when that depends on the arguments."""
    global LAUNCHES
    fn = getattr(lib, name)
    prof = _PROFILE
    if prof is not None and (prof.get('__only__') is None or name in prof['__only__']):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        code = fn(*args)
        e1.record()
        prof.setdefault(name, []).append((e0, e1))
    else:
        code = fn(*args)
    check(code, name)
    LAUNCHES += kernels if kernels is not None else _KERNELS_PER_CALL.get(name, 1)


class profile_ops:
    """Context manager: CUDA-event timing around every entry point (or only the named ones) on the current stream.
    After the block (and a synchronize) `times_ms()` gives name -> list of durations."""

    def __init__(self, only=None):
        self.records = {'__only__': set(only) if only else None}

    def __enter__(self):
        global _PROFILE
        self._prev, _PROFILE = _PROFILE, self.records
        return self

    def __exit__(self, *exc):
        global _PROFILE
        _PROFILE = self._prev
        return False

    def times_ms(self):
        torch.cuda.synchronize()
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in self.records.items() if k != '__only__'}


def _chk(t: Tensor, name: str, dtype=torch.float32) -> Tensor:
    if not isinstance(t, Tensor):
        raise TypeError(f'{name} must be a torch.Tensor')
    if not t.is_cuda:
        raise ValueError(f'{name} must be a CUDA tensor (spgt_b200 has no CPU path)')
    if t.dtype != dtype:
        raise TypeError(f'{name} must be {dtype}, got {t.dtype}')
    if not t.is_contiguous():
        raise ValueError(f'{name} must be contiguous')
    return t


def _p(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------------------------------------
# attention ops
# ---------------------------------------------------------------------------------------------------------
def projpos(x: Tensor, weight: Tensor, bias: Optional[Tensor], position: Tensor, num_head: int, dim_head: int,
            dim_position: int) -> Tensor:
    _chk(x, 'input'); _chk(weight, 'weight'); _chk(position, 'position')
    if bias is not None:
        _chk(bias, 'bias')
    B, S, D = x.shape
    out = torch.empty(B, num_head, dim_position + dim_head, S, device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _call('spgt_projpos_fwd', x.data_ptr(), weight.data_ptr(), _p(bias), position.data_ptr(), out.data_ptr(),
                                   B, S, D, num_head, dim_head, dim_position, _stream())
    return out


def projpos_lnorm(x: Tensor, weight: Tensor, bias: Optional[Tensor], ln_weight: Tensor, ln_bias: Tensor,
                  position: Tensor, norm_eps: float, num_head: int, dim_head: int, dim_position: int,
                  return_invsigma: bool = False):
    _chk(x, 'input'); _chk(weight, 'weight'); _chk(position, 'position'); _chk(ln_weight, 'ln_weight'); _chk(ln_bias, 'ln_bias')
    if bias is not None:
        _chk(bias, 'bias')
    B, S, D = x.shape
    out = torch.empty(B, num_head, dim_position + dim_head, S, device=x.device, dtype=x.dtype)
    inv = torch.empty(B, num_head, S, device=x.device, dtype=x.dtype) if return_invsigma else None
    with torch.cuda.device(x.device):
        _call('spgt_projpos_lnorm_fwd', x.data_ptr(), weight.data_ptr(), _p(bias), ln_weight.data_ptr(), ln_bias.data_ptr(),
                                         float(norm_eps), position.data_ptr(), out.data_ptr(), _p(inv),
                                         B, S, D, num_head, dim_head, dim_position, _stream())
    return (out, inv) if return_invsigma else out


def projpos_qkv(x, wq, bq, wk, bk, wv, bv, lnwk, lnbk, lnwv, lnbv, eps, position, num_head, dim_head, dim_position):
    for n, t in (('x', x), ('wq', wq), ('wk', wk), ('wv', wv), ('position', position)):
        _chk(t, n)
    B, S, D = x.shape
    q, k, v = (torch.empty(B, num_head, dim_position + dim_head, S, device=x.device, dtype=x.dtype) for _ in range(3))
    with torch.cuda.device(x.device):
        _call('spgt_projpos_qkv_fwd', x.data_ptr(), wq.data_ptr(), _p(bq), wk.data_ptr(), _p(bk), wv.data_ptr(), _p(bv),
                                       lnwk.data_ptr(), lnbk.data_ptr(), lnwv.data_ptr(), lnbv.data_ptr(), float(eps),
                                       position.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                       B, S, D, num_head, dim_head, dim_position, _stream())
    return q, k, v


def galerkin_attention(Q: Tensor, K: Tensor, V: Tensor, merged_heads: bool = False, return_kv: bool = False):
    _chk(Q, 'Q'); _chk(K, 'K'); _chk(V, 'V')
    if Q.dim() != 4 or Q.shape != K.shape or Q.shape != V.shape:
        raise ValueError('Q, K, V must share the shape [batch, num_head, d_posk, seqlen]')
    B, H, dpk, S = Q.shape
    shape = (B, S, H * dpk) if merged_heads else (B, H, S, dpk)
    out = torch.empty(shape, device=Q.device, dtype=Q.dtype)
    T = torch.empty(B, H, dpk, dpk, device=Q.device, dtype=Q.dtype) if return_kv else None
    with torch.cuda.device(Q.device):
        _call('spgt_galerkin_attn_fwd', Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), _p(T),
                                         B, H, dpk, S, int(merged_heads), _stream())
    return (out, T) if return_kv else out


def projpos_backward(x: Tensor, weight: Tensor, bias: Optional[Tensor], ln_weight: Optional[Tensor], grad_out: Tensor,
                     norm_eps: float, num_head: int, dim_head: int, dim_position: int):
    """Gradients of projpos (ln_weight None) or projpos_lnorm with respect to (x, weight, bias, ln_weight, ln_bias) for
    grad_out [B, H, dim_position + dim_head, S].  The element-wise stage (gather, LayerNorm backward, parameter sums) is
    one kernel; dX = dh W^T and dW = x^T dh reuse the tcgen05 linear and the transpose + split-K skinny GEMM."""
    _chk(x, 'input'); _chk(weight, 'weight'); _chk(grad_out, 'grad_out')
    B, S, D = x.shape
    if grad_out.shape != (B, num_head, dim_position + dim_head, S) or D != num_head * dim_head:
        raise ValueError('shape mismatch')
    x2 = x.reshape(B * S, D)
    h = linear_tc(x2, TcWeight(weight), bias) if ln_weight is not None else None
    dh = torch.empty(B * S, D, device=x.device, dtype=x.dtype)
    db = torch.empty(D, device=x.device, dtype=x.dtype)
    dlnw = torch.empty(D, device=x.device, dtype=x.dtype) if ln_weight is not None else None
    dlnb = torch.empty(D, device=x.device, dtype=x.dtype) if ln_weight is not None else None
    need = int(lib.spgt_projpos_bwd_workspace_bytes(B, S, num_head))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _call('spgt_projpos_bwd_elementwise', grad_out.data_ptr(), _p(h), _p(ln_weight), float(norm_eps), dh.data_ptr(), db.data_ptr(),
              _p(dlnw), _p(dlnb), B, S, num_head, dim_head, dim_position, ws.data_ptr(), need, _stream())
    dx = linear_tc(dh, TcWeight(weight.t().contiguous()), None).view(B, S, D)
    xT = batched_transpose(x2, [1], [B * S], [D])                       # [1, D, rows]
    dW = batched_skinny_gemm(xT, dh.view(1, B * S, D), 1.0).view(D, D)
    shape = ln_weight.shape if ln_weight is not None else None
    return dx, dW, db, (dlnw.view(shape) if dlnw is not None else None), (dlnb.view(shape) if dlnb is not None else None)


def galerkin_attention_backward(Q: Tensor, K: Tensor, V: Tensor, grad_out: Tensor):
    """Gradients (dQ, dK, dV), each [B,H,dpk,S], of galerkin_attention(Q, K, V) -> [B,H,S,dpk] for grad_out [B,H,S,dpk]."""
    for t, n in ((Q, 'Q'), (K, 'K'), (V, 'V'), (grad_out, 'grad_out')):
        _chk(t, n)
    B, H, dpk, S = Q.shape
    if K.shape != Q.shape or V.shape != Q.shape or grad_out.shape != (B, H, S, dpk):
        raise ValueError('shape mismatch')
    need = int(lib.spgt_galerkin_attn_bwd_workspace_bytes(B, H, dpk, S))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=Q.device)
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(Q), torch.empty_like(Q)
    with torch.cuda.device(Q.device):
        _call('spgt_galerkin_attn_bwd', Q.data_ptr(), K.data_ptr(), V.data_ptr(), grad_out.data_ptr(), dQ.data_ptr(), dK.data_ptr(),
              dV.data_ptr(), B, H, dpk, S, ws.data_ptr(), need, _stream())
    return dQ, dK, dV


def relative_l2(pred: Tensor, target: Tensor, eps: float = 1.0e-10) -> Tensor:
    """Per-sample relative L2 error of [N, ...] tensors (engine/metric.py:47-67 of the reference): [N]."""
    pred, target = _chk(pred.contiguous(), 'pred'), _chk(target.contiguous(), 'target')
    if pred.shape != target.shape:
        raise ValueError('pred and target must have the same shape')
    N = pred.shape[0]
    out = torch.empty(N, dtype=torch.float32, device=pred.device)
    _call('spgt_relative_l2_fwd', pred.data_ptr(), target.data_ptr(), out.data_ptr(), N, pred.numel() // N, float(eps), _stream())
    return out


def darcy_fv_solve(coef_nodes: Tensor, f_nodes: Tensor, rel_tol: float = 1.0e-10, max_iter: int = 20000,
                   check_every: int = 100):
    """Solve the finite-volume Darcy system of the reference's generator (dataset/darcy_generate/Solve_GWF.m:16-38) for
    a batch of node coefficient fields: float64 CUDA tensors [B, K, K] in, (p [B, K, K], iterations, relative residuals
    [B]) out.  Raises if the conjugate-gradient iteration does not reach rel_tol within max_iter."""
    for t, n in ((coef_nodes, 'coef_nodes'), (f_nodes, 'f_nodes')):
        if not (t.is_cuda and t.dtype == torch.float64):
            raise ValueError(f'{n} must be a float64 CUDA tensor')
    coef_nodes, f_nodes = coef_nodes.contiguous(), f_nodes.contiguous()
    if coef_nodes.dim() != 3 or coef_nodes.shape[1] != coef_nodes.shape[2] or coef_nodes.shape != f_nodes.shape:
        raise ValueError('coef_nodes and f_nodes must both be [B, K, K]')
    B, K = coef_nodes.shape[0], coef_nodes.shape[1]
    p = torch.empty_like(coef_nodes)
    ws = torch.empty(int(lib.spgt_darcy_fv_workspace_bytes(B, K)), dtype=torch.uint8, device=coef_nodes.device)
    iters = ctypes.c_int(0)
    rel = (ctypes.c_double * B)()
    _call('spgt_darcy_fv_solve', coef_nodes.data_ptr(), f_nodes.data_ptr(), p.data_ptr(), B, K, int(max_iter), float(rel_tol),
          int(check_every), ws.data_ptr(), ws.numel(), ctypes.addressof(iters), ctypes.addressof(rel), _stream())
    return p, iters.value, list(rel)


def skinny_gemm_workspace_bytes(M: int, N: int, K: int, batch: int) -> int:
    return int(lib.spgt_skinny_gemm_workspace_bytes(M, N, K, batch))


def batched_skinny_gemm(A: Tensor, Bm: Tensor, alpha: float = 1.0, workspace: Optional[Tensor] = None) -> Tensor:
    _chk(A, 'A'); _chk(Bm, 'B')
    if A.dim() < 2 or A.dim() != Bm.dim() or A.shape[:-2] != Bm.shape[:-2] or A.shape[-1] != Bm.shape[-2]:
        raise ValueError('A must be [..., M, K] and B [..., K, N] with equal batch dims')
    M, K, N = A.shape[-2], A.shape[-1], Bm.shape[-1]
    batch = int(math.prod(A.shape[:-2]))
    Cm = torch.empty(*A.shape[:-2], M, N, device=A.device, dtype=A.dtype)
    need = skinny_gemm_workspace_bytes(M, N, K, batch)
    if workspace is None:
        workspace = torch.empty(need, device=A.device, dtype=torch.uint8)
    with torch.cuda.device(A.device):
        _call('spgt_batched_skinny_gemm', A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), float(alpha), M, N, K, batch,
                                           workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream())
    return Cm


# ---------------------------------------------------------------------------------------------------------
# data movement
# ---------------------------------------------------------------------------------------------------------
def batched_transpose(X: Tensor, batch_list: Sequence[int], M_list: Sequence[int], N_list: Sequence[int]) -> Tensor:
    _chk(X, 'X')
    b, M, N = math.prod(batch_list), math.prod(M_list), math.prod(N_list)
    if X.numel() != b * M * N:
        raise ValueError('X does not have prod(batch)*prod(M)*prod(N) elements')
    out = torch.empty(*batch_list, *N_list, *M_list, device=X.device, dtype=X.dtype)
    with torch.cuda.device(X.device):
        _call('spgt_batched_transpose', X.data_ptr(), out.data_ptr(), M, N, b, _stream())
    return out


def transpose_gather_dual(src: Tensor, dim_list, H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2) -> Tuple[Tensor, Tensor]:
    _chk(src, 'src', torch.complex64)
    dim = math.prod(dim_list)
    if src.numel() != dim * H_all * W_all:
        raise ValueError('src does not have prod(dim)*H_all*W_all elements')
    o1 = torch.empty(H_low, W_low, *dim_list, device=src.device, dtype=src.dtype)
    o2 = torch.empty_like(o1)
    with torch.cuda.device(src.device):
        _call('spgt_transpose_gather_dual', src.data_ptr(), o1.data_ptr(), o2.data_ptr(), dim, H_all, W_all, H_low, W_low,
                                             hb1, wb1, hb2, wb2, _stream())
    return o1, o2


def transpose_scatter_dual(src1: Tensor, src2: Tensor, dim_list, H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2) -> Tensor:
    _chk(src1, 'src1', torch.complex64); _chk(src2, 'src2', torch.complex64)
    dim = math.prod(dim_list)
    if src1.numel() != dim * H_low * W_low or src2.numel() != src1.numel():
        raise ValueError('src1/src2 do not have H_low*W_low*prod(dim) elements')
    out = torch.empty(*dim_list, H_all, W_all, device=src1.device, dtype=src1.dtype)
    with torch.cuda.device(src1.device):
        _call('spgt_transpose_scatter_dual', src1.data_ptr(), src2.data_ptr(), out.data_ptr(), dim, H_all, W_all,
                                              H_low, W_low, hb1, wb1, hb2, wb2, _stream())
    return out


# ---------------------------------------------------------------------------------------------------------
# dense layers
# ---------------------------------------------------------------------------------------------------------
def pad_cols(w: Tensor, multiple: int = 4) -> Tensor:
    """[K, N] -> contiguous [K, ceil(N/multiple)*multiple] with zero columns appended (kernel weight pitch rule)."""
    K, N = w.shape
    Np = (N + multiple - 1) // multiple * multiple
    if Np == N:
        return w.contiguous()
    out = torch.zeros(K, Np, device=w.device, dtype=w.dtype)
    out[:, :N] = w
    return out


def linear(x: Tensor, w_kn: Tensor, bias: Optional[Tensor], N: int, act=None, residual: Optional[Tensor] = None,
           out: Optional[Tensor] = None) -> Tensor:
    """y = act(x @ w_kn[:, :N] + bias) (+ residual).  x [..., K] contiguous, w_kn [K, ldw] (ldw % 4 == 0)."""
    _chk(x, 'x'); _chk(w_kn, 'weight')
    K = x.shape[-1]
    rows = x.numel() // K
    if w_kn.shape[0] != K:
        raise ValueError('weight must be [K, ldw]')
    if out is None:
        out = torch.empty(*x.shape[:-1], N, device=x.device, dtype=x.dtype)
    if residual is not None:
        _chk(residual, 'residual')
    with torch.cuda.device(x.device):
        _call('spgt_linear_fwd', x.data_ptr(), K, w_kn.data_ptr(), w_kn.shape[1], _p(bias), _p(residual), N,
                                  out.data_ptr(), N, rows, K, N, act_code(act), _stream())
    return out


def conv3x3(x: Tensor, cin_off: int, Cin: int, w_kn: Tensor, bias: Tensor, y: Tensor, cout_off: int, Cout: int, act) -> Tensor:
    """NHWC 3x3 convolution reading channels [cin_off, cin_off+Cin) of x and writing [cout_off, cout_off+Cout) of y."""
    _chk(x, 'x'); _chk(w_kn, 'weight'); _chk(y, 'y'); _chk(bias, 'bias')
    B, Hh, Ww, cp = x.shape
    if y.shape[:3] != x.shape[:3]:
        raise ValueError('x and y must share [B, H, W]')
    with torch.cuda.device(x.device):
        _call('spgt_conv3x3_fwd', x.data_ptr(), cp, cin_off, Cin, w_kn.data_ptr(), w_kn.shape[1], bias.data_ptr(),
                                   y.data_ptr(), y.shape[3], cout_off, Cout, B, Hh, Ww, act_code(act), _stream())
    return y


def bilinear(x: Tensor, Ho: int, Wo: int, act=None) -> Tensor:
    _chk(x, 'x')
    B, Hi, Wi, Cc = x.shape
    y = torch.empty(B, Ho, Wo, Cc, device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _call('spgt_bilinear_fwd', x.data_ptr(), y.data_ptr(), B, Hi, Wi, Ho, Wo, Cc, act_code(act), _stream())
    return y


def bilinear_concat3(x1: Tensor, x2: Tensor, x3: Tensor, c1: int, c2: int, c3: int, Ho: int, Wo: int, act=None) -> Tensor:
    """act(bilinear(concat(x1[..., :c1], x2[..., :c2], x3[..., :c3]))) -> [B, Ho, Wo, c1+c2+c3]."""
    _chk(x1, 'x1'); _chk(x2, 'x2'); _chk(x3, 'x3')
    B, Hi, Wi, _ = x1.shape
    y = torch.empty(B, Ho, Wo, c1 + c2 + c3, device=x1.device, dtype=x1.dtype)
    with torch.cuda.device(x1.device):
        _call('spgt_bilinear_concat3_fwd', x1.data_ptr(), x2.data_ptr(), x3.data_ptr(), x1.shape[3], x2.shape[3], x3.shape[3],
              c1, c2, c3, y.data_ptr(), B, Hi, Wi, Ho, Wo, act_code(act), _stream())
    return y


def conv0_down(node: Tensor, w9: Tensor, bias: Tensor, Ho: int, Wo: int, act) -> Tensor:
    """node [B,Hi,Wi] (one channel), w9 [9, Cout] -> act(bilinear(act(conv3x3)))  [B,Ho,Wo,Cout]."""
    _chk(node, 'node'); _chk(w9, 'weight'); _chk(bias, 'bias')
    B, Hi, Wi = node.shape
    Cout = w9.shape[1]
    y = torch.empty(B, Ho, Wo, Cout, device=node.device, dtype=node.dtype)
    with torch.cuda.device(node.device):
        _call('spgt_conv0_down_fwd', node.data_ptr(), w9.data_ptr(), bias.data_ptr(), y.data_ptr(), B, Hi, Wi, Ho, Wo, Cout,
                                      act_code(act), _stream())
    return y


def upsample_grid(uw: Tensor, grid: Tensor, wg: Tensor, bias: Tensor, Ho: int, Wo: int) -> Tensor:
    _chk(uw, 'uw'); _chk(grid, 'grid'); _chk(wg, 'wg'); _chk(bias, 'bias')
    B, Hi, Wi, Cc = uw.shape
    y = torch.empty(B, Ho, Wo, Cc, device=uw.device, dtype=uw.dtype)
    with torch.cuda.device(uw.device):
        _call('spgt_upsample_grid_fwd', uw.data_ptr(), grid.data_ptr(), wg.data_ptr(), bias.data_ptr(), y.data_ptr(),
                                         B, Hi, Wi, Ho, Wo, Cc, _stream())
    return y


def decoder_head(x: Tensor, w1_kn: Tensor, b1: Tensor, w2: Tensor, b2: float, scale: float, shift: float,
                 dirichlet: bool, act, scale_map: Optional[Tensor] = None, shift_map: Optional[Tensor] = None) -> Tensor:
    """x [B,H,W,K] -> [B,H,W,1]: ((act(x@w1+b1) . w2) + b2) * scale + shift with an optional zero frame.
    scale_map / shift_map [H*W] replace the scalars per grid node when given."""
    _chk(x, 'x'); _chk(w1_kn, 'w1'); _chk(b1, 'b1'); _chk(w2, 'w2')
    B, Hh, Ww, K = x.shape
    out = torch.empty(B, Hh, Ww, 1, device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _call('spgt_decoder_head_fwd', x.data_ptr(), w1_kn.data_ptr(), b1.data_ptr(), w2.data_ptr(), float(b2), float(scale),
                                        float(shift), _p(scale_map), _p(shift_map), int(dirichlet), out.data_ptr(), B, Hh, Ww, K, w1_kn.shape[1],
                                        act_code(act), _stream())
    return out


# ---------------------------------------------------------------------------------------------------------
# tcgen05 / TMEM variants of the dense layers
# ---------------------------------------------------------------------------------------------------------
class TcWeight:
    """A [K, N] weight prepared for the tcgen05 kernels (tf32 hi/lo planes, K-major, padded)."""

    def __init__(self, w_kn: Tensor):
        _chk(w_kn, 'weight')
        self.K, self.N = w_kn.shape
        n = int(lib.spgt_tc_weight_bytes(self.K, self.N))
        self.buf = torch.empty(n, dtype=torch.uint8, device=w_kn.device)
        with torch.cuda.device(w_kn.device):
            _call('spgt_tc_weight_prepare', w_kn.data_ptr(), w_kn.shape[1], self.K, self.N, self.buf.data_ptr(), n, _stream())

    def data_ptr(self) -> int:
        return self.buf.data_ptr()


def tc_status() -> int:
    """0, or the code of the first bounded wait of a tensor-core kernel that gave up since the last reset (synchronises)."""
    return int(lib.spgt_tc_status())


def check_tc_status(where: str) -> None:
    """Raise (and clear the latched code) if a kernel gave up on a wait: its outputs are incomplete and must be discarded.
    Host loops call this at their synchronisation points."""
    code = tc_status()
    if code != 0:
        lib.spgt_tc_status_reset()
        raise RuntimeError(f'{where}: a tensor-core kernel gave up on a bounded wait (code {code}); results since the last check are invalid')


def linear_tc(x: Tensor, w: TcWeight, bias: Optional[Tensor], act=None, residual: Optional[Tensor] = None) -> Tensor:
    _chk(x, 'x')
    K = x.shape[-1]
    if K != w.K:
        raise ValueError('x last dim must equal the prepared weight K')
    rows = x.numel() // K
    out = torch.empty(*x.shape[:-1], w.N, device=x.device, dtype=x.dtype)
    if residual is not None:
        _chk(residual, 'residual')
    with torch.cuda.device(x.device):
        _call('spgt_linear_tc_fwd', x.data_ptr(), K, w.data_ptr(), _p(bias), _p(residual), w.N, out.data_ptr(), w.N,
              rows, K, w.N, act_code(act), _stream())
    return out


def ffn_tc(x: Tensor, w1: TcWeight, b1: Tensor, w2: TcWeight, b2: Optional[Tensor], act, residual: Optional[Tensor] = None) -> Tensor:
    """act(x W1 + b1) W2 + b2 (+ residual) in one kernel; x [..., 128], W1 [128, 256], W2 [256, 128]."""
    _chk(x, 'x'); _chk(b1, 'b1')
    D = x.shape[-1]
    if D != w1.K or w1.N != w2.K or w2.N != D:
        raise ValueError('prepared weights do not chain: need W1 [D, H] and W2 [H, D]')
    rows = x.numel() // D
    out = torch.empty_like(x)
    if residual is not None:
        _chk(residual, 'residual')
    with torch.cuda.device(x.device):
        _call('spgt_ffn_tc_fwd', x.data_ptr(), D, w1.data_ptr(), b1.data_ptr(), w2.data_ptr(), _p(b2), _p(residual), D,
              out.data_ptr(), D, rows, D, w1.N, act_code(act), _stream())
    return out


def conv3x3_tc(x: Tensor, cin_off: int, Cin: int, w: TcWeight, bias: Tensor, y: Tensor, cout_off: int, Cout: int, act) -> Tensor:
    _chk(x, 'x'); _chk(y, 'y'); _chk(bias, 'bias')
    B, Hh, Ww, cp = x.shape
    if w.K != 9 * Cin or w.N != Cout:
        raise ValueError('prepared weight does not match [9*Cin, Cout]')
    with torch.cuda.device(x.device):
        _call('spgt_conv3x3_tc_fwd', x.data_ptr(), cp, cin_off, Cin, w.data_ptr(), bias.data_ptr(), y.data_ptr(), y.shape[3],
              cout_off, Cout, B, Hh, Ww, act_code(act), _stream())
    return y


def projpos_qkv_tc(x, wqkv: TcWeight, bq, bk, bv, lnwk, lnbk, lnwv, lnbv, eps, position, num_head, dim_head, dim_position):
    _chk(x, 'x'); _chk(position, 'position')
    B, S, D = x.shape
    q, k, v = (torch.empty(B, num_head, dim_position + dim_head, S, device=x.device, dtype=x.dtype) for _ in range(3))
    with torch.cuda.device(x.device):
        _call('spgt_projpos_qkv_tc_fwd', x.data_ptr(), wqkv.data_ptr(), _p(bq), _p(bk), _p(bv), lnwk.data_ptr(), lnbk.data_ptr(),
              lnwv.data_ptr(), lnbv.data_ptr(), float(eps), position.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
              B, S, D, num_head, dim_head, dim_position, _stream())
    return q, k, v


def decoder_head_tc(x: Tensor, w1: TcWeight, b1: Tensor, w2: Tensor, b2: float, scale: float, shift: float, dirichlet: bool,
                    act, scale_map: Optional[Tensor] = None, shift_map: Optional[Tensor] = None) -> Tensor:
    _chk(x, 'x'); _chk(b1, 'b1'); _chk(w2, 'w2')
    B, Hh, Ww, K = x.shape
    out = torch.empty(B, Hh, Ww, 1, device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _call('spgt_decoder_head_tc_fwd', x.data_ptr(), w1.data_ptr(), b1.data_ptr(), w2.data_ptr(), float(b2), float(scale),
              float(shift), _p(scale_map), _p(shift_map), int(dirichlet), out.data_ptr(), B, Hh, Ww, K, w1.N,
              act_code(act), _stream())
    return out


# ---------------------------------------------------------------------------------------------------------
# spectral layer
# ---------------------------------------------------------------------------------------------------------
_TABLES = {}


def spectral_tables(r: int, m: int, device) -> Tensor:
    """DFT tables for (r, m), computed once per device by a setup kernel and cached."""
    key = (r, m, torch.device(device).index)
    if key not in _TABLES:
        n = int(lib.spgt_spectral_tables_bytes(r, m))
        if n == 0:
            raise ValueError(f'unsupported spectral shape r={r}, m={m}')
        t = torch.empty(n, device=device, dtype=torch.uint8)
        with torch.cuda.device(device):
            _call('spgt_spectral_tables_init', t.data_ptr(), n, r, m, _stream())
        _TABLES[key] = t
    return _TABLES[key]


def spectral_conv2d(x: Tensor, wr_kn: Tensor, br: Tensor, fw0: Tensor, fw1: Tensor, mode: int, act,
                    workspace: Optional[Tensor] = None) -> Tensor:
    """x [B,r,r,32]; wr_kn [32,32] = residual weight transposed; fw0/fw1 [m,m,32,32,2]."""
    _chk(x, 'x'); _chk(wr_kn, 'wr'); _chk(br, 'br'); _chk(fw0, 'fw0'); _chk(fw1, 'fw1')
    B, r, r2, Cc = x.shape
    if r != r2:
        raise ValueError('the spectral layer expects a square grid')
    tab = spectral_tables(r, mode, x.device)
    need = int(lib.spgt_spectral_workspace_bytes(B, r, mode, Cc))
    if need == 0:
        raise ValueError(f'unsupported spectral shape B={B} r={r} m={mode} C={Cc}')
    if workspace is None:
        workspace = torch.empty(need, device=x.device, dtype=torch.uint8)
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _call('spgt_spectral_conv2d_fwd', x.data_ptr(), wr_kn.data_ptr(), br.data_ptr(), fw0.data_ptr(), fw1.data_ptr(),
                                           tab.data_ptr(), workspace.data_ptr(), workspace.numel(), y.data_ptr(),
                                           B, r, Cc, mode, act_code(act), _stream(),
              kernels=int(lib.spgt_spectral_launches(B, r, mode)))
    return y
