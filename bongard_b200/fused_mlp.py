"""Pre-norm + gated MLP as one module, with the reference's fused_mlp call surface.

Mirrors bongard/fused_mlp.py: `enable_fused_mlp(model, recipe)` replaces every text layer's
`mlp` by a module that also owns the pre-feed-forward RMSNorm (zero-centred gain) and sets
`layer.pre_feedforward_layernorm` to Identity (fused_mlp.py:84-98), returning the count.
The module keeps the native parameter objects, so `hf_state_dict` only has to rename keys.
"""

from __future__ import annotations

import torch
from torch import nn

from . import ops
from .te_linear import RECIPES, B200MLP, _layers


class B200FusedMLP(nn.Module):
    """y = MLP(rmsnorm(x) * (1 + w)): RMSNorm kernel, GEMM + GeGLU epilogue, GEMM."""

    def __init__(self, mlp, norm, recipe='bf16'):
        super().__init__()
        self.bongard_recipe = recipe
        self.layer_norm_weight, self.eps = norm.weight, norm.eps
        self.intermediate_size = mlp.intermediate_size
        self.mlp = B200MLP(mlp, recipe)

    def forward(self, x):
        if self.training and torch.is_grad_enabled() and (x.requires_grad or self.layer_norm_weight.requires_grad):
            # train mode: norm and projections record their backward kernels
            return self.mlp(ops.rmsnorm_autograd(x, self.layer_norm_weight, self.eps))
        n = ops.rmsnorm(x if x.stride(-1) == 1 else x.contiguous(), self.layer_norm_weight.detach().to(torch.bfloat16),
                        self.eps)
        return self.mlp(n)


def enable_fused_mlp(model, recipe='bf16'):
    if recipe not in RECIPES:
        raise ValueError(f'Fused MLP requires one of the recipes {RECIPES}')
    ops.device_check()
    count = 0
    for layer in _layers(model):
        if isinstance(layer.mlp, B200FusedMLP):
            if layer.mlp.bongard_recipe != recipe:
                raise ValueError('An existing fused MLP must retain its recipe')
        else:
            layer.mlp = B200FusedMLP(layer.mlp, layer.pre_feedforward_layernorm, recipe)
            layer.pre_feedforward_layernorm = nn.Identity()
        count += 1
    return count


def hf_state_dict(module_name, fused: B200FusedMLP):
    """Hugging Face keys for one fused MLP (the inverse of the stacking, bongard/fused_mlp.py:101-124)."""
    layer = module_name.rsplit('.', 1)[0]
    gate, up = fused.mlp.gate_up.weight.split(fused.intermediate_size)
    return {f'{layer}.pre_feedforward_layernorm.weight': fused.layer_norm_weight,
            f'{module_name}.gate_proj.weight': gate, f'{module_name}.up_proj.weight': up,
            f'{module_name}.down_proj.weight': fused.mlp.down.weight}
