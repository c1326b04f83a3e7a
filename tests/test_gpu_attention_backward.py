"""Backward of the packed attention against autograd through the fp32 oracle: encoder (global and
sliding window), decoder with a state prefix (causal, windowed), GQA, head sizes 64 and 256."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import ops  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'


def rnd(*shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).bfloat16()


def oracle_grads(q, k, v, dout, lengths, scale, window, cross=None, owners=None, state_lengths=None):
    leaves = [t.float().requires_grad_(True) for t in (q, k, v)]
    cr = None
    if cross is not None:
        cr = tuple(t.float().requires_grad_(True) for t in cross)
        leaves += list(cr)
    out, _ = om.varlen_attention(leaves[0], leaves[1], leaves[2], lengths, scale, window, cross=cr, owners=owners,
                                 state_lengths=state_lengths)
    out.backward(dout.float().view_as(out))
    return out.detach(), [t.grad for t in leaves]


def check(got, want, name):
    got, want = got.float().cpu(), want.float()
    assert got.shape == want.shape, name
    assert torch.isfinite(got).all(), name
    scale = float(want.abs().max()) + 1e-6
    err = float((got - want).abs().max()) / scale
    assert err < 2e-2, f'{name}: max err {err:.4g} of the largest gradient'


@pytest.mark.parametrize('d,hq,hkv', [(64, 4, 2), (256, 8, 4), (64, 2, 2)])
@pytest.mark.parametrize('lengths,window', [([70, 200, 1, 129], None), ([300, 64, 513], 128), ([257], 33)])
def test_encoder_backward(d, hq, hkv, lengths, window):
    t = sum(lengths)
    q, k, v, dout = rnd(t, hq, d, seed=1), rnd(t, hkv, d, seed=2), rnd(t, hkv, d, seed=3), rnd(t, hq, d, seed=4)
    scale = d ** -0.5
    _, want = oracle_grads(q, k, v, dout, lengths, scale, window)
    plan = ops.make_plan(lengths, window, DEV, group=hq // hkv, head_dim=d, backward=True)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = ops.varlen_attention_autograd(qd, kd, vd, plan, scale)
    out.backward(dout.to(DEV).view_as(out))
    ops.read_status()
    for got, ref, name in zip((qd.grad, kd.grad, vd.grad), want, ('dq', 'dk', 'dv')):
        check(got, ref, name)


@pytest.mark.parametrize('d,hq,hkv', [(64, 4, 2), (256, 8, 4)])
@pytest.mark.parametrize('window', [None, 24])
def test_decoder_backward_with_state_prefix(d, hq, hkv, window):
    lengths = [40, 17, 90, 130, 5]
    owners = [0, 0, 1, 2, 2]
    state_lengths = [150, 64, 300, 20]            # the last state has no question: zero gradient
    t, ts = sum(lengths), sum(state_lengths)
    q, k, v, dout = rnd(t, hq, d, seed=5), rnd(t, hkv, d, seed=6), rnd(t, hkv, d, seed=7), rnd(t, hq, d, seed=8)
    ck, cv = rnd(ts, hkv, d, seed=9), rnd(ts, hkv, d, seed=10)
    scale = d ** -0.5
    _, want = oracle_grads(q, k, v, dout, lengths, scale, window, (ck, cv), owners, state_lengths)
    want[3] = torch.zeros_like(ck.float()) if want[3] is None else want[3]
    plan = ops.make_plan(lengths, window, DEV, group=hq // hkv, owners=owners, state_lengths=state_lengths, head_dim=d,
                         backward=True)
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k, v, ck, cv)]
    out = ops.varlen_attention_autograd(leaves[0], leaves[1], leaves[2], plan, scale, (leaves[3], leaves[4]))
    out.backward(dout.to(DEV).view_as(out))
    ops.read_status()
    for leaf, ref, name in zip(leaves, want, ('dq', 'dk', 'dv', 'dck', 'dcv')):
        check(leaf.grad, ref, name)
    assert float(leaves[3].grad[-20:].abs().max()) == 0 and float(leaves[4].grad[-20:].abs().max()) == 0


def test_backward_is_deterministic_and_rejects_split_owners():
    lengths, d, hq, hkv = [200, 333], 64, 4, 2
    t = sum(lengths)
    q, k, v, dout = (rnd(t, h, d, seed=s).to(DEV) for h, s in ((hq, 11), (hkv, 12), (hkv, 13), (hq, 14)))
    plan = ops.make_plan(lengths, None, DEV, group=2, head_dim=d, backward=True)
    out, lse = ops.varlen_attention(q, k, v, plan, 0.125, return_lse=True)
    a = ops.varlen_attention_backward(q, k, v, plan, 0.125, out, lse, dout)
    b = ops.varlen_attention_backward(q, k, v, plan, 0.125, out, lse, dout)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    with pytest.raises(ValueError, match='consecutive'):
        ops.make_host_plan([10, 10, 10], None, group=2, owners=[0, 1, 0], state_lengths=[5, 5], backward=True)
    with pytest.raises(ValueError, match='key tiles'):
        ops.varlen_attention_backward(q, k, v, ops.make_plan(lengths, None, DEV, group=2, head_dim=d), 0.125, out, lse, dout)
