"""Parity of every CUDA entry point (called through the C ABI) against the CPU oracle.

Tolerances: bf16 attention / MLP / linear outputs within 2e-2 absolute + 1e-2 relative of the
fp32 oracle evaluated on the same bf16-rounded inputs; glue kernels within one bf16 rounding.
"""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import ops  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'
ATOL, RTOL = 2e-2, 1e-2


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).bfloat16()


def assert_close(got, want, atol=ATOL, rtol=RTOL):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    if got.numel() == 0:
        return
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    worst = float((err - bound).max())
    assert worst <= 0, f'max abs err {float(err.max()):.4g}, exceeds bound by {worst:.4g}'


@pytest.fixture(scope='module', autouse=True)
def device():
    ops.device_check()
    yield
    ops.read_status()


@pytest.mark.parametrize('rows,h', [(1, 256), (7, 256), (33, 2560), (5000, 2560), (5, 8192), (6, 264), (0, 256)])
def test_rmsnorm(rows, h):
    x, w = rnd(rows, h, seed=1), rnd(h, seed=2, std=0.2)
    got = ops.rmsnorm(x.to(DEV), w.to(DEV))
    want = om.rmsnorm(x.float(), w.float())
    assert_close(got, want, atol=1e-2, rtol=8e-3)


@pytest.mark.parametrize('rows,h', [(9, 256), (40, 2560), (3000, 2560), (11, 264)])
def test_add_rmsnorm(rows, h):
    y, resid = rnd(rows, h, seed=3), rnd(rows, h, seed=4)
    wp, wn = rnd(h, seed=5, std=0.2), rnd(h, seed=6, std=0.2)
    r = resid.to(DEV).clone()
    normed = ops.add_rmsnorm_(y.to(DEV), wp.to(DEV), r, wn.to(DEV))
    want_r = resid + om.rmsnorm(y, wp)          # bf16 chain, as the module sequence computes it
    want_n = om.rmsnorm(want_r, wn)
    assert_close(r, want_r, atol=1.6e-2, rtol=8e-3)      # one bf16 step of the post-norm value, where a rounding tie falls the other way
    assert_close(normed, want_n, atol=1e-2, rtol=8e-3)
    r2 = resid.to(DEV).clone()
    assert ops.add_rmsnorm_(y.to(DEV), wp.to(DEV), r2, None) is None
    assert torch.equal(r2, r)


@pytest.mark.parametrize('rows,h', [(1, 256), (1037, 2560), (70000, 256), (3, 4096), (0, 512)])
def test_fp32_residual_stream(rows, h):
    """The residual stream kept in fp32: the norms read it, the update adds the post-norm result without
    rounding, the embedding writes it unrounded.  Against the oracle's fp32 arithmetic on the same inputs."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(rows, h, generator=g) * 3
    y, wp, wn = rnd(rows, h, seed=13), rnd(h, seed=14, std=0.2), rnd(h, seed=15, std=0.2)
    got = ops.rmsnorm(x.to(DEV), wp.to(DEV))
    assert got.dtype == torch.bfloat16
    assert_close(got, om.rmsnorm(x, wp.float()), atol=1e-2, rtol=8e-3)
    r = x.to(DEV).clone()
    normed = ops.add_rmsnorm_(y.to(DEV), wp.to(DEV), r, wn.to(DEV))
    want_r = x + om.rmsnorm(y.float(), wp.float())
    assert r.dtype == torch.float32 and normed.dtype == torch.bfloat16
    assert_close(r, want_r, atol=1e-5, rtol=1e-5)            # nothing rounded on the way into the stream
    assert_close(normed, om.rmsnorm(want_r, wn.float()), atol=1e-2, rtol=8e-3)
    r2 = x.to(DEV).clone()
    assert ops.add_rmsnorm_(y.to(DEV), wp.to(DEV), r2, None) is None and torch.equal(r2, r)
    if h % 256 == 0 and rows:
        with pytest.raises(ValueError):
            ops.rmsnorm(torch.zeros(2, 264, device=DEV), torch.zeros(264, device=DEV, dtype=torch.bfloat16))


def test_embed_fp32():
    table, eoi = rnd(300, 256, seed=10, std=0.02), rnd(256, seed=11, std=0.1)
    ids = torch.tensor([5, 123, 299, 0, 123, 17])
    scale = math.sqrt(256)
    got = ops.embed(ids.to(DEV), table.to(DEV), eoi.to(DEV), scale, eoi_token=123, dtype=torch.float32)
    want = table.float()[ids] * scale
    want[ids == 123] = eoi.float()
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)


@pytest.mark.parametrize('d,hq,hkv,theta', [(64, 4, 2, 1e4), (256, 8, 4, 1e6), (256, 8, 4, 1e4), (128, 2, 1, 1e4)])
def test_qk_norm_rope(d, hq, hkv, theta):
    lengths = [5, 130, 1, 700]
    t = sum(lengths)
    qkv = rnd(t, (hq + 2 * hkv) * d, seed=7)
    qw, kw = rnd(d, seed=8, std=0.2), rnd(d, seed=9, std=0.2)
    positions = torch.cat([torch.arange(n) for n in lengths])
    buf = qkv.to(DEV).clone()
    q = buf[:, :hq * d].view(t, hq, d)
    k = buf[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    ops.qk_norm_rope_(q, k, qw.to(DEV), kw.to(DEV), positions.int().to(DEV), ops.inv_freq(d, theta, DEV))
    cos, sin = om.rope_tables(positions, d, theta, torch.float32)
    wq, wk = om.qk_norm_rope(qkv[:, :hq * d].float().view(t, hq, d), qkv[:, hq * d:(hq + hkv) * d].float().view(t, hkv, d),
                             qw.float(), kw.float(), cos, sin)
    assert_close(q, wq, atol=1.5e-2, rtol=8e-3)
    assert_close(k, wk, atol=1.5e-2, rtol=8e-3)
    assert torch.equal(buf[:, (hq + hkv) * d:].cpu(), qkv[:, (hq + hkv) * d:])   # v untouched
    # angles from the per-position table: the same bits as the angles computed per token
    buf3 = qkv.to(DEV).clone()
    q3 = buf3[:, :hq * d].view(t, hq, d)
    k3 = buf3[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    ops.qk_norm_rope_(q3, k3, qw.to(DEV), kw.to(DEV), positions.int().to(DEV), None,
                      table=ops.rope_table(d, theta, max(lengths), DEV))
    assert torch.equal(buf3, buf)
    # normalise only (decoder state keys)
    buf2 = qkv.to(DEV).clone()
    k2 = buf2[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    ops.qk_norm_rope_(None, k2, None, kw.to(DEV), None, None, rotate=False)
    assert_close(k2, om.rmsnorm(qkv[:, hq * d:(hq + hkv) * d].float().view(t, hkv, d), kw.float()), atol=1e-2, rtol=8e-3)
    assert torch.equal(buf2[:, :hq * d].cpu(), qkv[:, :hq * d])


def test_embed():
    table, eoi = rnd(300, 256, seed=10, std=0.02), rnd(256, seed=11, std=0.1)
    ids = torch.tensor([5, 123, 299, 0, 123, 17])
    scale = float(torch.tensor(math.sqrt(256)).bfloat16())
    got = ops.embed(ids.to(DEV), table.to(DEV), eoi.to(DEV), scale, eoi_token=123)
    want = om.embed(ids, table, eoi, 256, eoi_token=123)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize('m,n,k', [(1, 256, 256), (129, 512, 256), (300, 2560, 1024), (1000, 4096, 2560),
                                   (77, 264, 72), (4096, 2560, 10240)])
def test_linear(m, n, k):
    x, w = rnd(m, k, seed=12), rnd(n, k, seed=13, std=0.02)
    got = ops.linear(x.to(DEV), w.to(DEV))
    want = x.float() @ w.float().t()
    assert_close(got, want)


def test_linear_strided_input_and_output():
    x = rnd(200, 1024, seed=14)
    w = rnd(512, 256, seed=15, std=0.05)
    xd = x.to(DEV)
    out = torch.zeros(200, 1024, device=DEV, dtype=torch.bfloat16)
    ops.linear(xd[:, 256:512], w.to(DEV), out=out[:, 512:])
    assert_close(out[:, 512:], x[:, 256:512].float() @ w.float().t())
    assert float(out[:, :512].abs().max()) == 0


@pytest.mark.parametrize('m,i,k', [(5, 1024, 256), (300, 1024, 256), (1500, 10240, 2560)])
def test_linear_geglu(m, i, k):
    x = rnd(m, k, seed=16)
    gate, up = rnd(i, k, seed=17, std=0.02), rnd(i, k, seed=18, std=0.02)
    got = ops.linear_geglu(x.to(DEV), torch.cat([gate, up]).to(DEV))
    want = torch.nn.functional.gelu(x.float() @ gate.float().t(), approximate='tanh') * (x.float() @ up.float().t())
    assert_close(got, want)


# the four projections of a 4B layer and of the tiny model, at row counts around the 128-row tiles
@pytest.mark.parametrize('n,k', [(4096, 2560), (2560, 2048), (2560, 10240), (512, 256), (256, 1024)])
@pytest.mark.parametrize('m', [1, 100, 128, 129, 256])
def test_linear_few_rows(m, n, k):
    """The split-K weight-streaming kernel against fp32 and against the throughput kernel."""
    x, w = rnd(m, k, seed=30), rnd(n, k, seed=31, std=0.02)
    xd, wd = x.to(DEV), w.to(DEV)
    got = ops.linear(xd, wd, few_rows=True)
    assert_close(got, x.float() @ w.float().t())
    # same products, another fp32 summation order: equal up to one rounding of the bf16 result
    assert_close(got, ops.linear(xd, wd).float(), atol=2e-3, rtol=8e-3)
    assert torch.equal(got, ops.linear(xd, wd, few_rows=True))          # deterministic reduction


@pytest.mark.parametrize('m,i,k', [(3, 1024, 256), (140, 10240, 2560), (256, 10240, 2560), (200, 1024, 256)])
def test_linear_geglu_few_rows(m, i, k):
    x = rnd(m, k, seed=32)
    gate, up = rnd(i, k, seed=33, std=0.02), rnd(i, k, seed=34, std=0.02)
    got = ops.linear_geglu(x.to(DEV), torch.cat([gate, up]).to(DEV), few_rows=True)
    want = torch.nn.functional.gelu(x.float() @ gate.float().t(), approximate='tanh') * (x.float() @ up.float().t())
    assert_close(got, want)


def test_linear_few_rows_falls_back_and_entry_point_rejects():
    """Shapes the kernel does not take run on the throughput kernels; the entry point itself says no."""
    from bongard_b200 import _lib

    x, w = rnd(300, 256, seed=35).to(DEV), rnd(384, 256, seed=36, std=0.05).to(DEV)
    assert_close(ops.linear(x, w, few_rows=True), x.float().cpu() @ w.float().cpu().t())      # 300 rows
    assert_close(ops.linear(x[:8, :200], w[:128, :200].contiguous(), few_rows=True),            # k % 64 != 0
                 x[:8, :200].float().cpu() @ w[:128, :200].float().cpu().t())
    lib = _lib.load()
    assert lib.bg_gemm_bf16_skinny_supported(256, 384, 256, 0) == 1
    assert lib.bg_gemm_bf16_skinny_supported(257, 384, 256, 0) == 0
    assert lib.bg_gemm_bf16_skinny_supported(8, 200, 256, 0) == 0
    out = torch.empty(300, 384, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        _lib.check(lib.bg_gemm_bf16_skinny(x.data_ptr(), 256, w.data_ptr(), 256, out.data_ptr(), 384, 300, 384, 256, 0, 0),
                   'bg_gemm_bf16_skinny')


@pytest.mark.parametrize('d,hq,hkv,theta', [(64, 4, 2, 1e4), (256, 8, 4, 1e6), (128, 2, 2, 1e4)])
@pytest.mark.parametrize('m', [7, 300])
def test_qkv_projection_with_fused_norm_rope(d, hq, hkv, theta, m):
    """The q|k|v GEMM with QK-norm + RoPE in its epilogue against the two-kernel path (same rounding
    points, another summation order: a bf16 ulp at most) and against the fp32 oracle."""
    k_in, qd, kd = 256, hq * d, hkv * d
    x, w = rnd(m, k_in, seed=40), rnd(qd + 2 * kd, k_in, seed=41, std=0.05)
    qw, kw = rnd(d, seed=42, std=0.1), rnd(d, seed=43, std=0.1)
    positions = (torch.arange(m, dtype=torch.int32) * 37) % 5000
    xd, wd, qwd, kwd, pd = (t.to(DEV) for t in (x, w, qw, kw, positions))
    table = ops.rope_table(d, theta, 5000, DEV)
    fused = ops.linear_qkv_rope(xd, wd, qd, kd, d, qwd, kwd, pd, table)
    plain = ops.linear(xd, wd)
    q, k = plain[:, :qd].view(m, hq, d), plain[:, qd:qd + kd].view(m, hkv, d)
    ops.qk_norm_rope_(q, k, qwd, kwd, pd, ops.inv_freq(d, theta, DEV))
    assert_close(fused, plain.float(), atol=2e-3, rtol=8e-3)
    assert torch.equal(fused[:, qd + kd:], plain[:, qd + kd:])                       # value heads untouched
    proj = (x.float() @ w.float().t()).bfloat16().float()
    cos, sin = om.rope_tables(positions.long(), d, theta, torch.float32)
    want_q, want_k = om.qk_norm_rope(proj[:, :qd].view(m, hq, d), proj[:, qd:qd + kd].view(m, hkv, d), qw.float(),
                                     kw.float(), cos, sin)
    assert_close(fused[:, :qd].view(m, hq, d), want_q, atol=3e-2, rtol=2e-2)
    assert_close(fused[:, qd:qd + kd].view(m, hkv, d), want_k, atol=3e-2, rtol=2e-2)


def test_geglu_mlp_matches_golden(golden_dir):
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items() if k.startswith('mlp_')}
    x = g['mlp_x'].bfloat16()
    gate_up = torch.cat([g['mlp_gate'], g['mlp_up']]).bfloat16()
    h = ops.linear_geglu(x.to(DEV), gate_up.to(DEV))
    y = ops.linear(h, g['mlp_down'].bfloat16().to(DEV))
    assert_close(y, g['mlp_y'])


def test_linear_rejects_bad_arguments():
    x, w = rnd(8, 256).to(DEV), rnd(256, 256).to(DEV)
    with pytest.raises(ValueError):
        ops.linear(x.float(), w)
    with pytest.raises(ValueError):
        ops.linear(x.cpu(), w.cpu())
    with pytest.raises(ValueError):
        ops.linear(x[:, :100], w[:, :100].contiguous())   # K not a multiple of 8


def test_judgment_head_and_softmax(golden_dir):
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items()}
    h, gg = g['head_h'].bfloat16(), g['head_g'][:1].bfloat16()
    hidden = torch.cat([h, gg]).to(DEV)
    cand = torch.arange(6, dtype=torch.int32, device=DEV)
    dec = torch.full((6,), 6, dtype=torch.int32, device=DEV)
    w, c, gr = (g[k].bfloat16() for k in ('head_w', 'head_c', 'head_gr'))
    logits = ops.judgment_head(hidden, cand, dec, w.to(DEV), c.to(DEV), gr.to(DEV))
    want = om.judgment_head(h.float(), gg.float().expand(6, -1), w.float(), c.float(), gr.float())
    assert_close(logits, want, atol=2e-4, rtol=1e-4)
    offsets = torch.tensor([0, 2, 6], dtype=torch.int32, device=DEV)
    for temp in (1.0, 0.5, 2.0):
        probs = ops.candidate_softmax(logits, offsets, temp).cpu()
        l = logits.cpu()
        want = torch.cat([om.probabilities(l[:2], temp), om.probabilities(l[2:], temp)])
        assert float((probs - want).abs().max()) < 1e-12


@pytest.mark.parametrize('m,n,k', [(5, 128, 64), (300, 512, 256), (1030, 2560, 2048)])
def test_linear_backward(m, n, k):
    """dx = dy W and dW = dy^T x through the tensor-core GEMM (operands transposed first) against autograd."""
    x, w, dy = rnd(m, k, seed=50), rnd(n, k, seed=51, std=0.05), rnd(m, n, seed=52)
    xd, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    ops.linear_autograd(xd, wd).backward(dy.to(DEV))
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xf @ wf.t()).backward(dy.float())
    assert_close(xd.grad, xf.grad, atol=2e-2, rtol=1e-2)
    assert_close(wd.grad, wf.grad, atol=2e-2 * (m ** 0.5), rtol=1e-2)
    t = ops.transpose(x.to(DEV))
    assert torch.equal(t[:, :m].cpu(), x.t()) and float(t[:, m:].abs().max() if t.shape[1] > m else 0) == 0


@pytest.mark.parametrize('keep', [True, False])
@pytest.mark.parametrize('m,i,k', [(7, 256, 128), (300, 1024, 256)])
def test_linear_geglu_backward(m, i, k, keep, monkeypatch):
    """Both training forms: pre-activations kept by the forward (plain GEMM + activation pass), or recomputed
    by the backward after the fused GEMM + GeGLU forward."""
    monkeypatch.setattr(ops, 'GEGLU_KEEP_PREACTIVATIONS', keep)
    x, gu, dh = rnd(m, k, seed=53), rnd(2 * i, k, seed=54, std=0.05), rnd(m, i, seed=55)
    xd, gd = x.to(DEV).requires_grad_(True), gu.to(DEV).requires_grad_(True)
    out = ops.linear_geglu_autograd(xd, gd)
    assert_close(out, ops.linear_geglu(x.to(DEV), gu.to(DEV)).float(), atol=2e-2, rtol=2e-2)
    out.backward(dh.to(DEV))
    xf, gf = x.float().requires_grad_(True), gu.float().requires_grad_(True)
    pre = xf @ gf.t()
    (torch.nn.functional.gelu(pre[:, :i], approximate='tanh') * pre[:, i:]).backward(dh.float())
    assert_close(xd.grad, xf.grad, atol=3e-2, rtol=2e-2)
    assert_close(gd.grad, gf.grad, atol=3e-2 * (m ** 0.5), rtol=2e-2)


@pytest.mark.parametrize('rows,h', [(1, 256), (7, 256), (700, 2560), (1300, 8192), (0, 256)])
def test_rmsnorm_backward(rows, h):
    """Input and gain gradients of the zero-centred RMSNorm against autograd of the oracle in fp32."""
    x, w, dy = rnd(rows, h, seed=60), rnd(h, seed=61, std=0.2), rnd(rows, h, seed=62)
    xd, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    ops.rmsnorm_autograd(xd, wd).backward(dy.to(DEV))
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    om.rmsnorm(xf, wf).backward(dy.float())
    assert xd.grad.dtype == torch.bfloat16 and wd.grad.dtype == torch.bfloat16
    assert_close(xd.grad, xf.grad, atol=1e-2, rtol=8e-3)
    assert_close(wd.grad, wf.grad, atol=1e-2 * max(rows, 1) ** 0.5, rtol=8e-3)
    # the fp32 gain gradient itself, and that a second run gives the same bits (no atomics)
    dx, dw = ops.rmsnorm_backward(x.to(DEV), w.to(DEV), dy.to(DEV))
    assert_close(dw, wf.grad, atol=2e-3 * max(rows, 1) ** 0.5, rtol=2e-3)
    dx2, dw2 = ops.rmsnorm_backward(x.to(DEV), w.to(DEV), dy.to(DEV))
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


@pytest.mark.parametrize('d,hq,hkv,theta', [(64, 4, 2, 1e4), (256, 8, 4, 1e6), (128, 2, 1, 1e4)])
def test_qk_norm_rope_backward(d, hq, hkv, theta):
    """Backward of QK-norm + RoPE (both angle sources, and the no-rotation form of the state keys)
    against autograd of the oracle in fp32."""
    lengths = [5, 130, 1, 700, 2300]
    t = sum(lengths)
    q, k = rnd(t, hq, d, seed=63), rnd(t, hkv, d, seed=64)
    qw, kw = rnd(d, seed=65, std=0.2), rnd(d, seed=66, std=0.2)
    dq, dk = rnd(t, hq, d, seed=67), rnd(t, hkv, d, seed=68)
    positions = torch.cat([torch.arange(n) for n in lengths])
    cos, sin = om.rope_tables(positions, d, theta, torch.float32)
    qf, kf, qwf, kwf = (v.float().requires_grad_(True) for v in (q, k, qw, kw))
    oq, ok = om.qk_norm_rope(qf, kf, qwf, kwf, cos, sin)
    torch.autograd.backward([oq, ok], [dq.float(), dk.float()])
    tol_w = 1e-2 * (t * hq) ** 0.5

    got = ops.qk_norm_rope_backward(q.to(DEV), k.to(DEV), qw.to(DEV), kw.to(DEV), dq.to(DEV), dk.to(DEV),
                                    positions=positions.int().to(DEV), freqs=ops.inv_freq(d, theta, DEV))
    assert_close(got[0], qf.grad, atol=1.5e-2, rtol=8e-3)
    assert_close(got[1], kf.grad, atol=1.5e-2, rtol=8e-3)
    assert_close(got[2], qwf.grad, atol=tol_w, rtol=8e-3)
    assert_close(got[3], kwf.grad, atol=tol_w, rtol=8e-3)
    again = ops.qk_norm_rope_backward(q.to(DEV), k.to(DEV), qw.to(DEV), kw.to(DEV), dq.to(DEV), dk.to(DEV),
                                      positions=positions.int().to(DEV), freqs=ops.inv_freq(d, theta, DEV))
    assert all(torch.equal(a, b) for a, b in zip(got, again))

    # bf16 tables through the autograd surface (strided q / k views of one projection output)
    cos16, sin16 = cos.bfloat16(), sin.bfloat16()
    qkv = torch.cat([q.reshape(t, -1), k.reshape(t, -1)], 1).to(DEV).requires_grad_(True)
    qwd, kwd = qw.to(DEV).requires_grad_(True), kw.to(DEV).requires_grad_(True)
    o = ops.qk_norm_rope_table_autograd(qkv[:, :hq * d].view(t, hq, d), qkv[:, hq * d:].view(t, hkv, d), qwd, kwd,
                                        cos16.to(DEV), sin16.to(DEV))
    torch.autograd.backward(list(o), [dq.to(DEV), dk.to(DEV)])
    qf2, kf2, qwf2, kwf2 = (v.float().requires_grad_(True) for v in (q, k, qw, kw))
    o2 = om.qk_norm_rope(qf2, kf2, qwf2, kwf2, cos16.float(), sin16.float())
    torch.autograd.backward(list(o2), [dq.float(), dk.float()])
    assert_close(o[0], o2[0], atol=1.5e-2, rtol=8e-3)
    assert_close(qkv.grad[:, :hq * d].view(t, hq, d), qf2.grad, atol=1.5e-2, rtol=8e-3)
    assert_close(qkv.grad[:, hq * d:].view(t, hkv, d), kf2.grad, atol=1.5e-2, rtol=8e-3)
    assert_close(qwd.grad, qwf2.grad, atol=tol_w, rtol=8e-3)
    assert_close(kwd.grad, kwf2.grad, atol=tol_w, rtol=8e-3)

    # normalise only, one tensor (the decoder's state keys)
    kf3, kwf3 = k.float().requires_grad_(True), kw.float().requires_grad_(True)
    om.rmsnorm(kf3, kwf3).backward(dk.float())
    dxk, none_k, dkw, none_w = ops.qk_norm_rope_backward(k.to(DEV), None, kw.to(DEV), None, dk.to(DEV), None, rotate=False)
    assert none_k is None and none_w is None
    assert_close(dxk, kf3.grad, atol=1e-2, rtol=8e-3)
    assert_close(dkw, kwf3.grad, atol=tol_w, rtol=8e-3)


@pytest.mark.parametrize('m,n,k', [(300, 2560, 10240), (640, 2560, 10240), (1000, 2560, 10240), (513, 1024, 4096),
                                   (700, 2048, 8200)])
def test_linear_split_k(m, n, k):
    """A few hundred rows against a narrow weight with a long contraction: K slices as extra work items of the
    CTA-pair kernel, fp32 partials summed once.  Against fp32, against the unsplit kernel, and repeatable."""
    from bongard_b200 import _lib

    lib = _lib.load()
    split = lib.bg_gemm_bf16_splitk_choice(m, n, k)
    assert split >= 2, 'the shape is meant to take the split-K path'
    x, w = rnd(m, k, seed=70), rnd(n, k, seed=71, std=0.02)
    xd, wd = x.to(DEV), w.to(DEV)
    got = ops.linear(xd, wd, few_rows=True)
    assert_close(got, x.float() @ w.float().t())
    assert_close(got, ops.linear(xd, wd).float(), atol=2e-3, rtol=8e-3)
    assert torch.equal(got, ops.linear(xd, wd, few_rows=True))
    # strided input and output views
    big = torch.zeros(m, n + 64, device=DEV, dtype=torch.bfloat16)
    wide = torch.cat([xd, xd], 1)
    ops.linear(wide[:, k:], wd, out=big[:, 64:], few_rows=True)
    assert torch.equal(big[:, 64:], got) and float(big[:, :64].abs().max()) == 0
    # the entry point's own checks
    work = torch.empty(lib.bg_gemm_bf16_splitk_workspace_bytes(m, n, split), device=DEV, dtype=torch.uint8)
    args = (xd.data_ptr(), k, wd.data_ptr(), k, got.data_ptr(), n, m, n, k)
    assert lib.bg_gemm_bf16_splitk(*args, split, work.data_ptr(), work.numel() - 16, None) == -5      # workspace
    assert lib.bg_gemm_bf16_splitk(*args, 1, work.data_ptr(), work.numel(), None) == -1               # split < 2
    assert lib.bg_gemm_bf16_splitk_choice(32768, 2560, 10240) == 1 and lib.bg_gemm_bf16_splitk_choice(640, 2560, 2048) == 1


@pytest.mark.parametrize('r,m,n', [(64, 256, 256), (1000, 512, 384), (5000, 2560, 1024), (777, 264, 136), (4096, 128, 4096)])
def test_linear_tn(r, m, n):
    """at.T @ wt with the contraction over the rows of both operands (MN-major tensor-core tiles) against fp32,
    and against the same product through explicit transposes."""
    at, wt = rnd(r, m, seed=80), rnd(r, n, seed=81, std=0.05)
    ad, wd = at.to(DEV), wt.to(DEV)
    got = ops.linear_tn(ad, wd)
    want = at.float().t() @ wt.float()
    assert_close(got, want, atol=2e-2 * (r ** 0.5) * 0.05 + 2e-2, rtol=1e-2)
    via = ops.linear(ops.transpose(ad), ops.transpose(wd))
    assert_close(got, via.float(), atol=2e-3 * float(want.abs().max()), rtol=8e-3)
    # strided views of wider tensors
    wide_a, wide_w = torch.cat([ad, ad], 1), torch.cat([wd, wd], 1)
    assert torch.equal(ops.linear_tn(wide_a[:, m:], wide_w[:, :n]), got)
    # a shape the entry point does not take falls back to transposes
    odd = ops.linear_tn(ad[:, :m - 4], wd)
    assert_close(odd, want[:m - 4], atol=2e-2 * (r ** 0.5) * 0.05 + 2e-2, rtol=1e-2)
