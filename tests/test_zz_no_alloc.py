"""The allocation-free FP8 linear (bg_linear_fp8_static) against the workspace-taking entry point.

Collected last on purpose: it exercises a library-internal buffer that every call shares, so it
runs after everything else and must pass both alone in a fresh process and after the other tests.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import _lib, ops  # noqa: E402

DEV = 'cuda'


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).bfloat16().to(DEV)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    ops.device_check()
    lib = _lib.load()
    assert lib.bg_linear_fp8_static_max_bytes() == 9 << 20
    w1 = ops.quantize_weight(rnd(512, 2560, seed=1, std=0.02))
    w2 = ops.quantize_weight(rnd(2 * 1024, 256, seed=2, std=0.02))      # [gate; up] for the GeGLU epilogue
    x1, x2 = rnd(700, 2560, seed=3), rnd(300, 256, seed=4)
    # two different calls back to back on one stream: the second reuses the buffer the first left dirty
    got1 = ops.linear_fp8_static(x1, w1)
    got2 = ops.linear_fp8_static(x2, w2, geglu=True)
    want1 = ops.linear_fp8(x1, w1)
    want2 = ops.linear_fp8(x2, w2, geglu=True)
    ops.read_status()
    # same kernels on the same quantised operands: identical results, far inside the 2e-2 + 1e-2 rel bound
    assert torch.equal(got1, want1)
    assert torch.equal(got2, want2)
    # and again, in the opposite order
    assert torch.equal(ops.linear_fp8_static(x2, w2, geglu=True), want2)
    assert torch.equal(ops.linear_fp8_static(x1, w1), want1)


def test_static_scratch_rejects_oversized_activations_clearly():
    w = ops.quantize_weight(rnd(128, 2560, seed=5, std=0.02))
    x = torch.zeros(4096, 2560, dtype=torch.bfloat16, device=DEV)       # 10 MiB of quantised activations > 9 MiB
    with pytest.raises(_lib.B200Error, match='built-in'):
        ops.linear_fp8_static(x, w)
    ops.read_status()
