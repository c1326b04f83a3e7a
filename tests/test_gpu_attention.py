"""Packed variable-length attention (C ABI) against the oracle and the reference's fixtures."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import ops  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).bfloat16()


def assert_close(got, want, atol=2e-2, rtol=1e-2):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    if got.numel() == 0:
        return
    err = (got - want).abs()
    worst = float((err - (atol + rtol * want.abs())).max())
    assert worst <= 0, f'max abs err {float(err.max()):.4g}, exceeds bound by {worst:.4g}'


@pytest.fixture(scope='module', autouse=True)
def device():
    ops.device_check()
    yield
    ops.read_status()


def run(q, k, v, lengths, scale, window, cross=None, owners=None, state_lengths=None, lse=False, pair=None):
    hq, hkv = q.shape[1], k.shape[1]
    plan = ops.make_plan(lengths, window, DEV, group=hq // hkv, owners=owners, state_lengths=state_lengths,
                         head_dim=q.shape[-1], pair=pair)
    cr = None if cross is None else (cross[0].to(DEV), cross[1].to(DEV))
    out = ops.varlen_attention(q.to(DEV), k.to(DEV), v.to(DEV), plan, scale, cr, return_lse=lse)
    if lse:
        return out[0].view(q.shape), out[1]
    return out.view(q.shape)


@pytest.mark.parametrize('window', [None, 4, 5, 16])
def test_encoder_golden(golden_dir, window):
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items() if k.startswith('att_')}
    q, k, v = (g[n].bfloat16() for n in ('att_q', 'att_k', 'att_v'))
    out = run(q, k, v, g['att_lengths'].tolist(), 0.125, window)
    assert_close(out, g[f'att_enc_w{window}'], atol=3e-2, rtol=2e-2)   # fixture inputs were fp32
    want, _ = om.varlen_attention(q.float(), k.float(), v.float(), g['att_lengths'].tolist(), 0.125, window)
    assert_close(out, want)


@pytest.mark.parametrize('window', [None, 4, 16])
def test_decoder_golden(golden_dir, window):
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items() if k.startswith('att_')}
    q, k, v, ck, cv = (g[n].bfloat16() for n in ('att_q', 'att_k', 'att_v', 'att_ck', 'att_cv'))
    lengths, owners, sl = g['att_lengths'].tolist(), g['att_owners'].tolist(), g['att_state_lengths'].tolist()
    out = run(q, k, v, lengths, 0.125, window, (ck, cv), owners, sl)
    assert_close(out, g[f'att_dec_w{window}'], atol=3e-2, rtol=2e-2)
    want, _ = om.varlen_attention(q.float(), k.float(), v.float(), lengths, 0.125, window,
                                  cross=(ck.float(), cv.float()), owners=owners, state_lengths=sl)
    assert_close(out, want)


@pytest.mark.parametrize('d,hq,hkv', [(64, 4, 2), (256, 8, 4), (256, 4, 4), (64, 8, 1)])
@pytest.mark.parametrize('window', [None, 1024, 37])
def test_encoder_random(d, hq, hkv, window):
    lengths = [1, 63, 64, 65, 127, 128, 129, 700, 1500, 2]
    t = sum(lengths)
    q, k, v = rnd(t, hq, d, seed=1), rnd(t, hkv, d, seed=2), rnd(t, hkv, d, seed=3)
    scale = d ** -0.5
    out, lse = run(q, k, v, lengths, scale, window, lse=True)
    want, want_lse = om.varlen_attention(q.float(), k.float(), v.float(), lengths, scale, window)
    assert_close(out, want)
    assert_close(lse, want_lse, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize('d,hq,hkv', [(256, 8, 4), (64, 4, 2)])
def test_many_short_items_per_persistent_cta(d, hq, hkv):
    """Thousands of work items with one or two key tiles each, mixed with a few long ones: every persistent CTA
    walks through many items whose first S is also their last, full and partial tiles alternate, and the
    barrier phases run on across all of them."""
    gen = torch.Generator().manual_seed(5)
    lengths = torch.randint(1, 150, (900,), generator=gen).tolist()
    for i in range(0, 900, 97):
        lengths[i] = 600 + i                       # a few items with 5 - 12 key tiles in between
    t = sum(lengths)
    q, k, v = rnd(t, hq, d, seed=21), rnd(t, hkv, d, seed=22), rnd(t, hkv, d, seed=23)
    scale = d ** -0.5
    out, lse = run(q, k, v, lengths, scale, None, lse=True)
    want, want_lse = om.varlen_attention(q.float(), k.float(), v.float(), lengths, scale, None)
    assert_close(out, want)
    assert_close(lse, want_lse, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize('d,hq,hkv', [(64, 4, 2), (256, 8, 4)])
@pytest.mark.parametrize('window', [None, 1024, 20])
def test_decoder_random(d, hq, hkv, window):
    state_lengths = [300, 1, 1000]
    owners = [0, 0, 0, 1, 2, 2, 2, 2, 0]
    lengths = [20, 141, 64, 33, 17, 130, 5, 90, 40]
    t, s = sum(lengths), sum(state_lengths)
    q, k, v = rnd(t, hq, d, seed=4), rnd(t, hkv, d, seed=5), rnd(t, hkv, d, seed=6)
    ck, cv = rnd(s, hkv, d, seed=7), rnd(s, hkv, d, seed=8)
    scale = d ** -0.5
    out = run(q, k, v, lengths, scale, window, (ck, cv), owners, state_lengths)
    want, _ = om.varlen_attention(q.float(), k.float(), v.float(), lengths, scale, window,
                                  cross=(ck.float(), cv.float()), owners=owners, state_lengths=state_lengths)
    assert_close(out, want)


@pytest.mark.parametrize('hq,hkv', [(4, 4), (8, 4), (8, 2), (8, 1)])
@pytest.mark.parametrize('window', [None, 300])
def test_cta_pair_and_single_cta_kernels_agree(hq, hkv, window, monkeypatch):
    """head_dim 256 has two forward kernels: 128-row tiles on single CTAs (the default) and 256-row tiles on
    CTA pairs (opt-in: pair=True, or ops.PAIR_ATTENTION, under which a forward-only plan cuts each run into full
    pair tiles plus, where the rest fits one CTA, a single-CTA tile).  All three tilings against the oracle,
    encoder and decoder, for every GQA group; segment lengths around the 64- and 128-token tile edges and an
    empty segment."""
    d = 256
    assert ops.make_plan([300], window, DEV, group=hq // hkv, head_dim=d).n_pair_tiles == 0    # single CTAs by default
    monkeypatch.setattr(ops, 'PAIR_ATTENTION', True)       # pair=None then cuts runs between the two kernels
    lengths = [1, 0, 64, 65, 127, 128, 129, 191, 193, 700, 1300]
    t = sum(lengths)
    q, k, v = rnd(t, hq, d, seed=21), rnd(t, hkv, d, seed=22), rnd(t, hkv, d, seed=23)
    scale = d ** -0.5
    want, want_lse = om.varlen_attention(q.float(), k.float(), v.float(), lengths, scale, window)
    for pair in (None, True, False):
        plan = ops.make_plan(lengths, window, DEV, group=hq // hkv, head_dim=d, pair=pair)
        assert (plan.n_pair_tiles > 0, plan.n_tiles > 0) == {True: (True, False), False: (False, True), None: (True, True)}[pair]
        out, lse = run(q, k, v, lengths, scale, window, lse=True, pair=pair)
        assert_close(out, want)
        assert_close(lse, want_lse, atol=2e-2, rtol=1e-3)
    state_lengths, owners = [300, 1, 1000, 0], [0, 0, 0, 1, 2, 2, 2, 2, 0, 3, 3]
    s = sum(state_lengths)
    ck, cv = rnd(s, hkv, d, seed=24), rnd(s, hkv, d, seed=25)
    want, _ = om.varlen_attention(q.float(), k.float(), v.float(), lengths, scale, window,
                                  cross=(ck.float(), cv.float()), owners=owners, state_lengths=state_lengths)
    for pair in (None, True, False):
        assert_close(run(q, k, v, lengths, scale, window, (ck, cv), owners, state_lengths, pair=pair), want)
    # a backward-capable plan keeps the 128-row tiles its passes are written for
    assert ops.make_plan(lengths, window, DEV, group=hq // hkv, head_dim=d, backward=True).n_pair_tiles == 0


def test_strided_qkv_views():
    """q, k, v as column blocks of one projection buffer, the layout the layer code uses."""
    d, hq, hkv = 256, 8, 4
    lengths = [200, 77]
    t = sum(lengths)
    qkv = rnd(t, (hq + 2 * hkv) * d, seed=9).to(DEV)
    q = qkv[:, :hq * d].view(t, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(t, hkv, d)
    plan = ops.make_plan(lengths, None, DEV, group=2, head_dim=d)
    out = ops.varlen_attention(q, k, v, plan, 1 / 16).view(t, hq, d)
    want, _ = om.varlen_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), lengths, 1 / 16, None)
    assert_close(out, want)


def test_large_scores_need_the_running_maximum():
    """Scores that grow along the key axis force repeated accumulator rescales."""
    d, hq, hkv = 64, 2, 1
    lengths = [900]
    q = rnd(900, hq, d, seed=10)
    k = rnd(900, hkv, d, seed=11) * torch.linspace(0.1, 6.0, 900)[:, None, None].bfloat16()
    v = rnd(900, hkv, d, seed=12)
    out = run(q, k, v, lengths, 1.0, None)
    want, _ = om.varlen_attention(q.float(), k.float(), v.float(), lengths, 1.0, None)
    assert_close(out, want)


def test_plan_tile_size_is_checked():
    lengths = [150, 70]
    t = sum(lengths)
    plan = ops.make_plan(lengths, None, DEV, group=2, head_dim=64)
    plan.tile_rows = 512          # a plan built for a larger tile than the kernel computes
    with pytest.raises(ValueError):
        ops.varlen_attention(rnd(t, 4, 64).to(DEV), rnd(t, 2, 64).to(DEV), rnd(t, 2, 64).to(DEV), plan, 0.125)


def test_rejects_unsupported_shapes():
    q, k = rnd(8, 3, 64).to(DEV), rnd(8, 1, 64).to(DEV)
    plan = ops.make_plan([8], None, DEV, group=2)
    with pytest.raises(ValueError):
        ops.varlen_attention(q, k, k, plan, 1.0)        # group of 3
    q = rnd(8, 2, 96).to(DEV)
    with pytest.raises(ValueError):
        ops.varlen_attention(q, rnd(8, 1, 96).to(DEV), rnd(8, 1, 96).to(DEV), plan, 1.0)   # head_dim 96
