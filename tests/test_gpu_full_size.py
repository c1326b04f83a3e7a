"""The op-level workloads at their full benchmark sizes (35 862 packed tokens of 16 sequences with
8 query / 4 KV heads of 256; 32 768 tokens through the 2560 -> 10240 -> 2560 MLP), checked through
properties that do not need an oracle of that size: sampled rows against the fp32 oracle (rows of a
linear layer and queries of an attention are independent), independence of a segment from the rest
of its pack, probabilities summing to one, exact scaling and column sums of the backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import ops, workload as wl  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'
HQ, HKV, D = 8, 4, 256
SCALE = D ** -0.5


def randn(*shape, seed, std=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * std).bfloat16()


@pytest.fixture(scope='module')
def packed():
    lengths = wl.varlen_lengths(2, 16)
    t = sum(lengths)
    assert t == 35862
    return lengths, randn(t, HQ, D, seed=1), randn(t, HKV, D, seed=2), randn(t, HKV, D, seed=3)


def oracle_rows(q, k, v, rows, lo, hi):
    """fp32 attention of single query rows against keys [lo, hi) of their segment."""
    out = []
    for r, a, b in zip(rows, lo, hi):
        qs = q[r].float().cpu().view(HKV, HQ // HKV, D)
        ks, vs = k[a:b].float().cpu(), v[a:b].float().cpu()
        s = torch.einsum('hgd,khd->hgk', qs, ks) * SCALE
        out.append(torch.einsum('hgk,khd->hgd', s.softmax(-1), vs).reshape(HQ * D))
    return torch.stack(out)


@pytest.mark.parametrize('window', [None, 1024])
def test_attention_full_size_sampled_rows_and_segment_independence(packed, window):
    lengths, q, k, v = packed
    plan = ops.make_plan(lengths, window, DEV, group=HQ // HKV, head_dim=D)
    out = ops.varlen_attention(q, k, v, plan, SCALE)
    ops.read_status()
    lo, hi = ops.plan_rows(lengths, window, decoder=False)
    rows = torch.randint(0, sum(lengths), (48,), generator=torch.Generator().manual_seed(5)).tolist() + [0, sum(lengths) - 1]
    want = oracle_rows(q, k, v, rows, lo[rows], hi[rows])
    assert float((out[rows].float().cpu() - want).abs().max()) < 2e-2
    # a segment's rows do not depend on what else is in the pack: bit-exact against a pack of one
    offset = 0
    for i, n in enumerate(lengths):
        if i in (2, 7, 15):
            alone = ops.varlen_attention(q[offset:offset + n], k[offset:offset + n], v[offset:offset + n],
                                         ops.make_plan([n], window, DEV, group=HQ // HKV, head_dim=D), SCALE)
            assert torch.equal(alone, out[offset:offset + n])
        offset += n
    # probabilities sum to one: with V = 1 every output is 1
    ones = ops.varlen_attention(q, k, torch.ones_like(v), plan, SCALE)
    assert float((ones.float() - 1).abs().max()) < 1e-2


def test_attention_backward_full_size_properties(packed):
    lengths, q, k, v = packed
    plan = ops.make_plan(lengths, None, DEV, group=HQ // HKV, head_dim=D, backward=True)
    out, lse = ops.varlen_attention(q, k, v, plan, SCALE, return_lse=True)
    dout = randn(sum(lengths), HQ, D, seed=4)
    dq, dk, dv = ops.varlen_attention_backward(q, k, v, plan, SCALE, out, lse, dout)
    ops.read_status()
    assert all(torch.isfinite(t.float()).all() for t in (dq, dk, dv))
    # every gradient row is written once, in a fixed order: a second run gives the same bits
    again = ops.varlen_attention_backward(q, k, v, plan, SCALE, out, lse, dout)
    assert all(torch.equal(a, b) for a, b in zip(again, (dq, dk, dv)))
    # doubling dout doubles every gradient: a power of two commutes with every rounding, so the results
    # agree bit for bit except where a vanishing probability's product leaves the flushed-to-zero range
    dq2, dk2, dv2 = ops.varlen_attention_backward(q, k, v, plan, SCALE, out, lse, dout * 2)
    for twice, once in ((dq2, dq), (dk2, dk), (dv2, dv)):
        a, b = twice.float(), once.float() * 2
        assert float((a == b).float().mean()) > 0.999
        assert float((a - b).abs().max()) <= 2 ** -7 * float(b.abs().max())
    # rows of P sum to one, so per segment and KV head the keys' dV sum to the queries' dO
    offset = 0
    for n in lengths:
        got = dv[offset:offset + n].float().sum(0)
        want = dout[offset:offset + n].float().view(n, HKV, HQ // HKV, D).sum((0, 2))
        assert float((got - want).abs().max()) < 0.02 * float(want.abs().max()) + 0.5
        offset += n
    # sampled rows of dq against autograd through the fp32 oracle on one short segment
    start, n = sum(lengths[:2]), lengths[2]
    sl = slice(start, start + n)
    leaves = [t[sl].float().cpu().requires_grad_(True) for t in (q, k, v)]
    o, _ = om.varlen_attention(*leaves, [n], SCALE, None)
    o.backward(dout[sl].float().cpu())
    for got, leaf in zip((dq[sl], dk[sl], dv[sl]), leaves):
        assert float((got.float().cpu() - leaf.grad).abs().max()) < 2e-2 * float(leaf.grad.abs().max())


def test_mlp_and_linears_full_size_sampled_rows():
    t, h, i = 32768, 2560, 10240
    x = randn(t, h, seed=11)
    gate, up, down = randn(i, h, seed=12, std=0.02), randn(i, h, seed=13, std=0.02), randn(h, i, seed=14, std=0.02)
    hidden = ops.linear_geglu(x, torch.cat([gate, up]))
    y = ops.linear(hidden, down)
    ops.read_status()
    rows = torch.randint(0, t, (64,), generator=torch.Generator().manual_seed(6)).tolist() + [0, t - 1]
    xs = x[rows].float().cpu()
    want_h = torch.nn.functional.gelu(xs @ gate.float().cpu().t(), approximate='tanh') * (xs @ up.float().cpu().t())
    assert float((hidden[rows].float().cpu() - want_h).abs().max()) < 2e-2 * float(want_h.abs().max())
    want_y = hidden[rows].float().cpu() @ down.float().cpu().t()
    assert float((y[rows].float().cpu() - want_y).abs().max()) < 1e-2 * float(want_y.abs().max()) + 1e-3
    # rows are independent: the same rows alone give the same bits
    assert torch.equal(ops.linear(ops.linear_geglu(x[1000:1300], torch.cat([gate, up])), down), y[1000:1300])
    # the E4M3 block-scaled path on the same inputs against its oracle on the sampled rows
    q_gu, q_down = ops.quantize_weight(torch.cat([gate, up])), ops.quantize_weight(down)
    h8 = ops.linear_fp8(x, q_gu, geglu=True)
    ops.read_status()
    want8 = om.geglu_mlp_fp8_block128(x[rows].cpu(), gate.cpu(), up.cpu(), down.cpu())
    y8 = ops.linear_fp8(h8, q_down)
    assert float((y8[rows].float().cpu() - want8.float()).abs().max()) < 3e-2 * float(want8.float().abs().max()) + 1e-3
    for name, n, k in (('qkv', 4096, 2560), ('o', 2560, 2048)):
        a, w = randn(t, k, seed=15), randn(n, k, seed=16, std=0.02)
        got = ops.linear(a, w)
        want = a[rows].float().cpu() @ w.float().cpu().t()
        assert float((got[rows].float().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max()) + 1e-3, name


@pytest.mark.parametrize('pair', [False, True])
def test_long_context_attention_sampled_rows(pair):
    """The long-context shape: one 32 768-token segment through the encoder kernel (global and window 1024) and a
    32 768-row state prefix in front of eight questions through the decoder form, on both forward kernels;
    sampled query rows against fp32 attention over exactly the keys each row may see."""
    n = 32768
    q, k, v = randn(n, HQ, D, seed=21), randn(n, HKV, D, seed=22), randn(n, HKV, D, seed=23)
    rows = torch.randint(0, n, (24,), generator=torch.Generator().manual_seed(7)).tolist() + [0, n - 1, 511, 512, n - 512]
    for window in (None, 1024):
        plan = ops.make_plan([n], window, DEV, group=HQ // HKV, head_dim=D, pair=pair)
        out = ops.varlen_attention(q, k, v, plan, SCALE)
        ops.read_status()
        lo, hi = ops.plan_rows([n], window, decoder=False)
        want = oracle_rows(q, k, v, rows, lo[rows], hi[rows])
        assert float((out[rows].float().cpu() - want).abs().max()) < 2e-2, window
    # decoder: every row of eight questions sees the whole state and its own causal prefix
    lengths = [141, 77, 200, 64, 129, 33, 180, 95]
    t = sum(lengths)
    qd, kd, vd = randn(t, HQ, D, seed=24), randn(t, HKV, D, seed=25), randn(t, HKV, D, seed=26)
    plan = ops.make_plan(lengths, None, DEV, group=HQ // HKV, owners=[0] * len(lengths), state_lengths=[n], head_dim=D, pair=pair)
    out = ops.varlen_attention(qd, kd, vd, plan, SCALE, (k, v))          # the segment's k, v serve as the state
    ops.read_status()
    starts = [sum(lengths[:i]) for i in range(len(lengths))]
    picks = [(0, 0), (0, 140), (3, 63), (7, 94), (4, 64), (6, 100)]
    for seg, pos in picks:
        r = starts[seg] + pos
        qs = qd[r].float().cpu().view(HKV, HQ // HKV, D)
        ks = torch.cat([k.float().cpu(), kd[starts[seg]:r + 1].float().cpu()])
        vs = torch.cat([v.float().cpu(), vd[starts[seg]:r + 1].float().cpu()])
        s = torch.einsum('hgd,khd->hgk', qs, ks) * SCALE
        want = torch.einsum('hgk,khd->hgd', s.softmax(-1), vs).reshape(HQ * D)
        assert float((out[r].float().cpu() - want).abs().max()) < 2e-2, (seg, pos)
