"""MXFP8 path (E4M3 with power-of-two scales per 32 K elements, scaled inside the tensor core):
quantisation bit-exact against the oracle, GEMM against the oracle's dequantised product."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import ops  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'


def rnd(*shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).bfloat16()


def scales_to_exponents(scales, rows, k):
    """Undo the 512-byte atom layout: int32 exponents [rows, K/32]."""
    s = scales.cpu().numpy().reshape(-1, k // 128, 32, 4, 4)          # [row atom][k atom][r % 32][r / 32][k sub-block]
    s = s.transpose(0, 3, 2, 1, 4).reshape(-1, k // 32)               # row = atom * 128 + (r / 32) * 32 + r % 32
    return torch.from_numpy(s[:rows].astype(np.int32) - 127)


@pytest.mark.parametrize('rows,k', [(1, 128), (130, 384), (300, 2560)])
def test_quantisation_is_bit_exact(rows, k):
    x = rnd(rows, k, seed=1, std=3.0)
    x[0, :32] = 0                                   # an all-zero block
    x[-1, -32:] *= 1e-30                            # a tiny block
    t = ops.quantize_mxfp8(x.to(DEV))
    q, e = om.quantize_mxfp8(x)
    assert torch.equal(scales_to_exponents(t.scales, rows, k), e)
    got = t.q.cpu().view(torch.float8_e4m3fn).float()
    assert torch.equal(got, q)


@pytest.mark.parametrize('m,n,k', [(128, 256, 128), (128, 256, 512), (1, 128, 128), (129, 512, 256), (300, 2560, 1024),
                                   (1000, 4096, 2560)])
def test_linear_mxfp8(m, n, k):
    x, w = rnd(m, k, seed=2), rnd(n, k, seed=3, std=0.05)
    wq = ops.quantize_mxfp8(w.to(DEV))
    got = ops.linear_mxfp8(x.to(DEV), wq)
    ops.read_status()
    want = om.linear_mxfp8(x, w)
    err = (got.float().cpu() - want.float()).abs()
    assert float(err.max()) <= 1e-2 * float(want.float().abs().max()) + 1e-3
    # the format itself costs a few percent against the unquantised product
    exact = x.float() @ w.float().t()
    assert float((got.float().cpu() - exact).abs().max()) < 0.08 * float(exact.abs().max())


@pytest.mark.parametrize('m,i,k', [(5, 1024, 256), (1500, 10240, 2560)])
def test_geglu_mxfp8(m, i, k):
    x = rnd(m, k, seed=4)
    gate, up, down = rnd(i, k, seed=5, std=0.02), rnd(i, k, seed=6, std=0.02), rnd(k, i, seed=7, std=0.02)
    h = ops.linear_mxfp8(x.to(DEV), ops.quantize_mxfp8(torch.cat([gate, up]).to(DEV)), geglu=True)
    y = ops.linear_mxfp8(h, ops.quantize_mxfp8(down.to(DEV)))
    ops.read_status()
    want = om.geglu_mlp_mxfp8(x, gate, up, down)
    assert float((y.float().cpu() - want.float()).abs().max()) <= 3e-2 * float(want.float().abs().max()) + 1e-3
