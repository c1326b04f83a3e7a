"""FP8 E4M3 block-scaled linears (C ABI) against the emulated oracle.

Two tolerances: (i) kernel vs the oracle's emulation of the same quantised operands must meet
the bf16 op bound (2e-2 abs + 1e-2 rel) because only accumulation order differs; (ii) the
quantisation error itself (emulation vs the unquantised product) is reported, not gated.
"""

import json

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
    assert got.shape == want.shape and torch.isfinite(got).all()
    err = (got - want).abs()
    worst = float((err - (atol + rtol * want.abs())).max())
    assert worst <= 0, f'max abs err {float(err.max()):.4g}, exceeds bound by {worst:.4g}'


@pytest.fixture(scope='module', autouse=True)
def device():
    ops.device_check()
    yield
    ops.read_status()


@pytest.mark.parametrize('m,k', [(1, 128), (5, 384), (300, 2560)])
def test_row_quantisation_is_bit_exact(m, k):
    x = rnd(m, k, seed=1) * 3
    q, inv = ops.quantize_rows(x.to(DEV))
    want_q, want_inv = om.quantize_e4m3_block(x.float(), 1, 128)
    assert torch.equal(q.cpu().view(torch.float8_e4m3fn).float(), want_q.float())
    assert torch.equal(inv.cpu().t(), want_inv)


@pytest.mark.parametrize('n,k', [(128, 128), (200, 256), (512, 2560)])
def test_tile_quantisation_is_bit_exact(n, k):
    w = rnd(n, k, seed=2, std=0.02)
    fw = ops.quantize_weight(w.to(DEV))
    want_q, want_inv = om.quantize_e4m3_block(w.float(), 128, 128)
    assert torch.equal(fw.q.cpu().view(torch.float8_e4m3fn).float(), want_q.float())
    assert torch.equal(fw.inv_scale.cpu(), want_inv)


@pytest.mark.parametrize('m,n,k', [(1, 128, 128), (129, 512, 256), (300, 2560, 1024), (1000, 4096, 2560),
                                   (700, 2560, 10240)])
def test_linear_fp8(m, n, k):
    x, w = rnd(m, k, seed=3), rnd(n, k, seed=4, std=0.02)
    got = ops.linear_fp8(x.to(DEV), ops.quantize_weight(w.to(DEV)))
    want = om.linear_fp8_block128(x.float(), w.float(), torch.float32)
    assert_close(got, want)
    exact = x.float() @ w.float().t()
    rel = float((want - exact).norm() / exact.norm())
    print(json.dumps(dict(m=m, n=n, k=k, relative_l2_quantisation_error=rel,
                          kernel_vs_emulation_max_abs=float((got.float().cpu() - want).abs().max()))))
    assert rel < 0.06


@pytest.mark.parametrize('m,i,k', [(5, 1024, 256), (1500, 10240, 2560)])
def test_geglu_fp8(m, i, k):
    x = rnd(m, k, seed=5)
    gate, up = rnd(i, k, seed=6, std=0.02), rnd(i, k, seed=7, std=0.02)
    got = ops.linear_fp8(x.to(DEV), ops.quantize_weight(torch.cat([gate, up]).to(DEV)), geglu=True)
    g = om.linear_fp8_block128(x.float(), gate.float(), torch.float32)
    u = om.linear_fp8_block128(x.float(), up.float(), torch.float32)
    assert_close(got, torch.nn.functional.gelu(g, approximate='tanh') * u)


def test_fp8_rejects_unaligned_k():
    x, w = rnd(8, 200).to(DEV), rnd(128, 256, std=0.02).to(DEV)
    with pytest.raises(ValueError):
        ops.quantize_rows(x)
    with pytest.raises(ValueError):
        ops.linear_fp8(rnd(8, 384).to(DEV), ops.quantize_weight(w))
