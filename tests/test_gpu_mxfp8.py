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


def test_engine_with_mxfp8_linears_stays_close_to_bf16():
    from bongard_b200 import workload as wl
    from bongard_b200.engine import JudgmentEngine

    weights = wl.make_weights(wl.TINY, 1, norm_std=0.1)
    requests = wl.tiny_requests(1)
    ref = torch.cat([p for a in JudgmentEngine(weights, wl.TINY).judge(requests) for p in a.values()])
    got = torch.cat([p for a in JudgmentEngine(weights, wl.TINY, linears='mxfp8').judge(requests) for p in a.values()])
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < 0.05


@pytest.mark.parametrize('m,i,k', [(5, 1024, 256), (700, 10240, 2560)])
def test_geglu_epilogue_emits_the_same_mxfp8_as_quantising_its_bf16_output(m, i, k):
    x = rnd(m, k, seed=8)
    gate_up = ops.quantize_mxfp8(rnd(2 * i, k, seed=9, std=0.02).to(DEV))
    a = ops.quantize_mxfp8(x.to(DEV))
    fused = ops.gemm_mxfp8_geglu_q(a, gate_up)
    two_pass = ops.quantize_mxfp8(ops.gemm_mxfp8(a, gate_up, geglu=True))
    ops.read_status()
    assert torch.equal(fused.q, two_pass.q) and torch.equal(fused.scales, two_pass.scales)


@pytest.mark.parametrize('rows,h', [(3, 256), (300, 2560)])
def test_norm_kernels_emit_the_same_mxfp8_as_quantising_their_bf16_output(rows, h):
    x, y = rnd(rows, h, seed=10).to(DEV), rnd(rows, h, seed=11).to(DEV)
    w1, w2 = rnd(h, seed=12, std=0.1).to(DEV), rnd(h, seed=13, std=0.1).to(DEV)
    a = ops.rmsnorm_mxfp8(x, w1)
    b = ops.quantize_mxfp8(ops.rmsnorm(x, w1))
    assert torch.equal(a.q, b.q) and torch.equal(a.scales, b.scales)
    r1, r2 = x.clone(), x.clone()
    c = ops.add_rmsnorm_mxfp8_(y, w1, r1, w2)
    d = ops.quantize_mxfp8(ops.add_rmsnorm_(y, w1, r2, w2))
    ops.read_status()
    assert torch.equal(r1, r2) and torch.equal(c.q, d.q) and torch.equal(c.scales, d.scales)


def test_converted_modules_with_the_mxfp8_recipe():
    """enable_te_linear / enable_fused_mlp with recipe 'mxfp8' on the Hugging Face backbone."""
    from bongard_b200 import workload as wl
    from bongard_b200.fused_mlp import enable_fused_mlp
    from bongard_b200.hf import build_backbone
    from bongard_b200.te_linear import enable_te_linear

    weights = wl.make_weights(wl.TINY, 1, norm_std=0.1)
    x = rnd(2, 40, wl.TINY.hidden, seed=20).to(DEV)
    with torch.no_grad():
        native = build_backbone(wl.TINY, weights)
        layer = native.decoder.layers[0]
        want = layer.mlp(layer.pre_feedforward_layernorm(x)).float()
        for convert in (lambda b: enable_te_linear(b, mlp='mxfp8'), lambda b: enable_fused_mlp(b, 'mxfp8')):
            backbone = build_backbone(wl.TINY, weights)
            convert(backbone)
            layer = backbone.decoder.layers[0]
            got = layer.mlp(layer.pre_feedforward_layernorm(x)).float()
            assert float((got - want).abs().max()) < 0.08 * float(want.abs().max())


def test_mxfp8_rejects_bad_shapes_and_handles_empty_input():
    w = ops.quantize_mxfp8(rnd(256, 256, seed=30).to(DEV))
    with pytest.raises(ValueError):
        ops.quantize_mxfp8(rnd(4, 200, seed=31).to(DEV))                     # K not a multiple of 128
    with pytest.raises(ValueError):
        ops.gemm_mxfp8(ops.quantize_mxfp8(rnd(4, 128, seed=32).to(DEV)), w)   # K mismatch
    empty = ops.linear_mxfp8(torch.zeros(0, 256, device=DEV, dtype=torch.bfloat16), w)
    assert empty.shape == (0, 256)
    # an all-zero activation quantises to zeros with the smallest scale and gives an all-zero product
    z = ops.linear_mxfp8(torch.zeros(3, 256, device=DEV, dtype=torch.bfloat16), w)
    assert float(z.abs().max()) == 0
