"""The tcgen05 / TMEM kernels against the oracle and against the warp-MMA kernels they replace."""
import pytest
import torch

from tests.helpers import load_golden, rel_l2
from oracle import gt_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope='module')
def dev():
    return torch.device('cuda:0')


@pytest.mark.parametrize('rows,K,N,act,res', [(128, 32, 32, None, False), (300, 128, 256, 'relu', False), (257, 256, 128, None, True),
                                              (1000, 136, 128, None, True), (5000, 128, 32, None, False), (77, 32, 44, 'silu', False),
                                              (40000, 128, 128, 'silu2', True), (1, 64, 64, None, False),
                                              # K > 256 (two row tiles per unit): 48-wide, 64-wide and 128-wide column tiles
                                              (700, 288, 44, 'silu', True), (515, 320, 36, None, False), (300, 288, 64, 'relu', False),
                                              (513, 384, 128, None, True)])
def test_linear_tc(dev, rows, K, N, act, res):
    from spgt_b200 import ops
    g = torch.Generator().manual_seed(rows + K)
    x, w, b = torch.randn(rows, K, generator=g), torch.randn(N, K, generator=g) / K ** 0.5, torch.randn(N, generator=g)
    r = torch.randn(rows, N, generator=g) if res else None
    wt = ops.TcWeight(w.t().contiguous().to(dev))
    y = ops.linear_tc(x.to(dev), wt, b.to(dev), act, None if r is None else r.to(dev))
    assert ops.tc_status() == 0
    ref = torch.nn.functional.linear(x.double(), w.double(), b.double())
    ref = {'relu': torch.relu, 'silu': torch.nn.functional.silu, None: lambda t: t,
           'silu2': lambda t: torch.nn.functional.silu(torch.nn.functional.silu(t))}[act](ref)
    if res:
        ref = ref + r.double()
    assert rel_l2(y, ref) < TOL
    assert torch.equal(y, ops.linear_tc(x.to(dev), wt, b.to(dev), act, None if r is None else r.to(dev)))


def test_bounded_wait_expires_and_status_latches(dev):
    """A wait on a barrier nothing arrives at gives up after its limit: the kernel returns, the code is latched until reset."""
    from spgt_b200 import ops
    from spgt_b200._lib import lib, check
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib.spgt_tc_selftest_wait_expiry(77, 500, flag.data_ptr(), torch.cuda.current_stream().cuda_stream), 'selftest')
    torch.cuda.synchronize()
    assert int(flag.item()) == 2                       # the wait expired and the thread went on
    assert ops.tc_status() == 77
    with pytest.raises(RuntimeError):
        ops.check_tc_status('test')
    assert ops.tc_status() == 0                        # check_tc_status clears the code after reporting it
    x = torch.randn(300, 128, device=dev)              # the context is still usable
    y = ops.linear_tc(x, ops.TcWeight(torch.eye(128, device=dev)), None)
    assert rel_l2(y, x.double().cpu()) < TOL and ops.tc_status() == 0


@pytest.mark.parametrize('B,Hh,Ww,cin_pitch,cin_off,Cin,Cout,act', [(2, 9, 11, 128, 0, 128, 44, 'relu'), (1, 13, 13, 132, 44, 44, 44, 'relu'),
                                                                    (1, 20, 17, 128, 0, 128, 128, 'silu2'), (2, 106, 106, 128, 0, 128, 128, 'silu2')])
def test_conv3x3_tc(dev, B, Hh, Ww, cin_pitch, cin_off, Cin, Cout, act):
    from spgt_b200 import ops
    g = torch.Generator().manual_seed(Cin + Cout)
    x = torch.randn(B, Hh, Ww, cin_pitch, generator=g)
    w = torch.randn(Cout, Cin, 3, 3, generator=g) / (9 * Cin) ** 0.5
    b = torch.randn(Cout, generator=g)
    wt = ops.TcWeight(w.permute(2, 3, 1, 0).reshape(9 * Cin, Cout).contiguous().to(dev))
    off = 4 if Cout + 4 <= 128 else 0
    y = torch.full((B, Hh, Ww, 128), float('nan'), device=dev)
    ops.conv3x3_tc(x.to(dev), cin_off, Cin, wt, b.to(dev), y, off, Cout, act)
    assert ops.tc_status() == 0
    ref = torch.nn.functional.conv2d(x[..., cin_off:cin_off + Cin].permute(0, 3, 1, 2).double(), w.double(), b.double(), padding=1)
    ref = torch.relu(ref) if act == 'relu' else torch.nn.functional.silu(torch.nn.functional.silu(ref))
    assert rel_l2(y[..., off:off + Cout], ref.permute(0, 2, 3, 1)) < TOL
    assert torch.isnan(y[..., :off]).all() and torch.isnan(y[..., off + Cout:]).all()


@pytest.mark.parametrize('B,S', [(1, 1), (2, 33), (3, 129), (2, 1849), (1, 2809)])
def test_projpos_qkv_tc(dev, B, S):
    from spgt_b200 import ops
    g = torch.Generator().manual_seed(S)
    x, pos = torch.randn(B, S, 128, generator=g), torch.rand(B, S, 2, generator=g)
    ws = [torch.randn(128, 128, generator=g) * 0.1 for _ in range(3)]
    bs = [torch.randn(128, generator=g) * 0.1 for _ in range(3)]
    lw, lb = 1 + 0.1 * torch.randn(2, 4, 32, generator=g), 0.1 * torch.randn(2, 4, 32, generator=g)
    wt = ops.TcWeight(torch.cat(ws, dim=1).contiguous().to(dev))
    q, k, v = ops.projpos_qkv_tc(x.to(dev), wt, bs[0].to(dev), bs[1].to(dev), bs[2].to(dev), lw[0].contiguous().to(dev),
                                 lb[0].contiguous().to(dev), lw[1].contiguous().to(dev), lb[1].contiguous().to(dev), 1e-6,
                                 pos.to(dev), 4, 32, 2)
    assert ops.tc_status() == 0
    d = lambda t: t.double()
    assert rel_l2(q, O.projpos(d(x), d(ws[0]), d(bs[0]), d(pos), 4, 32)) < TOL
    assert rel_l2(k, O.projpos_lnorm(d(x), d(ws[1]), d(bs[1]), d(lw[0]), d(lb[0]), d(pos), 1e-6, 4, 32)) < TOL
    assert rel_l2(v, O.projpos_lnorm(d(x), d(ws[2]), d(bs[2]), d(lw[1]), d(lb[1]), d(pos), 1e-6, 4, 32)) < TOL
    assert torch.equal(q[:, :, :2].cpu(), pos.transpose(1, 2).unsqueeze(1).expand(B, 4, 2, S))


def test_decoder_head_tc(dev):
    from spgt_b200 import ops
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 29, 29, 32, generator=g)
    w1, b1 = torch.randn(128, 32, generator=g) / 6, torch.randn(128, generator=g)
    w2, b2 = torch.randn(1, 128, generator=g) / 11, 0.3
    out = ops.decoder_head_tc(x.to(dev), ops.TcWeight(w1.t().contiguous().to(dev)), b1.to(dev), w2.reshape(-1).contiguous().to(dev),
                              b2, 1.00001, 0.5, True, 'silu')
    assert ops.tc_status() == 0
    h = torch.nn.functional.silu(torch.nn.functional.linear(x.double(), w1.double(), b1.double()))
    ref = (torch.nn.functional.linear(h, w2.double()) + b2) * 1.00001 + 0.5
    ref = torch.nn.functional.pad(ref[:, 1:-1, 1:-1], (0, 0, 1, 1, 1, 1))
    assert rel_l2(out, ref) < TOL


@pytest.mark.parametrize('rows,act,res', [(1, 'relu', False), (128, 'relu', True), (129, 'silu', True), (1000, 'relu', True),
                                          (64 * 2809, 'relu', True)])
def test_ffn_tc_fused(dev, rows, act, res):
    """The fused 128 -> 256 -> 128 feed-forward kernel against fp64, and bit-identical from run to run."""
    from spgt_b200 import ops
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 128, generator=g)
    w1, b1 = torch.randn(256, 128, generator=g) / 128 ** 0.5, torch.randn(256, generator=g)
    w2, b2 = torch.randn(128, 256, generator=g) / 256 ** 0.5, torch.randn(128, generator=g)
    t1, t2 = ops.TcWeight(w1.t().contiguous().to(dev)), ops.TcWeight(w2.t().contiguous().to(dev))
    xd = x.to(dev)
    y = ops.ffn_tc(xd, t1, b1.to(dev), t2, b2.to(dev), act, xd if res else None)
    assert ops.tc_status() == 0
    h = torch.nn.functional.linear(x.double(), w1.double(), b1.double())
    h = torch.relu(h) if act == 'relu' else torch.nn.functional.silu(h)
    ref = torch.nn.functional.linear(h, w2.double(), b2.double()) + (x.double() if res else 0.0)
    assert rel_l2(y, ref) < TOL
    assert torch.equal(y, ops.ffn_tc(xd, t1, b1.to(dev), t2, b2.to(dev), act, xd if res else None))
    two = ops.linear_tc(ops.linear_tc(xd, t1, b1.to(dev), act), t2, b2.to(dev), None, xd if res else None)
    assert rel_l2(y, two) < TOL
