"""FP8 text GEMMs with the reference's float8_training call surface.

Mirrors bongard/float8_training.py: `enable_float8(model, recipe, *, emulate=False)` converts
every bias-free text `nn.Linear` whose dimensions allow it and returns the count (27-65).
The reference's recipes are torchao's tensor-wise / row-wise dynamic scaling and only run in
train mode (eval serves F.linear, 20-21).  Here the recipe is 'block128': E4M3 operands with
dynamic per-call scales over 1 x 128 activation blocks and 128 x 128 weight tiles, and it runs
in inference.  `emulate=True` has no meaning without a CPU path and is rejected.
"""

from __future__ import annotations

import torch

from . import ops
from .te_linear import B200Linear

RECIPES = ('block128',)
# the reference's recipe names (bongard/float8_training.py:9): dynamic amax scaling per tensor / per row
REFERENCE_RECIPES = ('tensorwise', 'rowwise', 'rowwise_with_gw_hp')


def enable_float8(model, recipe='block128', *, emulate=False):
    """Convert every eligible text linear to the FP8 recipe and return the count (bongard/float8_training.py:27-65).

    Eligible: bias-free `nn.Linear` modules of the two text stacks whose dimensions are multiples of 128 (the
    reference asks for multiples of 16 and pads; 128 is the block this recipe scales by - every projection of the
    4B and tiny shapes qualifies).  The reference's own recipe names are refused with a message naming the
    replacement: its scaling granularities (one scale per tensor or per row) are coarser than 'block128' and
    there is no kernel for them here."""
    if recipe in REFERENCE_RECIPES:
        raise ValueError(f"recipe {recipe!r} (torchao dynamic scaling per tensor / per row) is served here by 'block128': the "
                         "same dynamic 448 / amax rule over 1 x 128 activation blocks and 128 x 128 weight tiles; pass "
                         "recipe='block128'")
    if recipe not in RECIPES:
        raise ValueError(f'fp8 must be one of {RECIPES}')
    if emulate:
        raise ValueError('bongard_b200 has no CPU emulation path; compare against oracle.reference_math instead')
    ops.device_check()
    backbone = model.backbone if hasattr(model, 'backbone') else model
    prefixes = ('encoder.text_model.layers.', 'decoder.layers.')
    count = 0
    for name, parent in list(backbone.named_modules()):
        if not name.startswith(prefixes):
            continue
        for child_name, child in list(parent.named_children()):
            if isinstance(child, B200Linear):
                if child.bongard_recipe != 'fp8':
                    raise ValueError('An already converted model must retain its recipe')
                continue
            if (isinstance(child, torch.nn.Linear) and child.bias is None
                    and child.in_features % 128 == 0 and child.out_features % 128 == 0):
                setattr(parent, child_name, B200Linear([child], 'fp8'))
                count += 1
    if not count:
        raise ValueError('FP8 found no eligible text Linear modules')
    return count
