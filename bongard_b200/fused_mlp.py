"""Pre-norm + gated MLP as one module, with the reference's fused_mlp call surface.

Mirrors bongard/fused_mlp.py: `enable_fused_mlp(model, recipe)` replaces every text layer's
`mlp` by a module that also owns the pre-feed-forward RMSNorm (zero-centred gain) and sets
`layer.pre_feedforward_layernorm` to Identity (fused_mlp.py:84-98), returning the count.
The norm gain and the down projection stay the native parameter objects; gate and up are stacked
into one parameter (as the reference's fc1_weight is, fused_mlp.py:37-38).  `hf_state_dict(backbone)`
gives the state under Hugging Face keys again, for `JudgmentModel.save` (bongard/model.py:531-539).
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


def hf_state_dict(backbone):
    """The backbone's state under Hugging Face keys, or None when nothing was converted
    (bongard/fused_mlp.py:101-124: the inverse of the fused gate/up layout and of the converted
    projections, what `Transformers.save_pretrained(state_dict=...)` is handed by JudgmentModel.save)."""
    from . import te_linear

    fused = [(name, module) for name, module in backbone.named_modules() if isinstance(module, B200FusedMLP)]
    if not fused and not te_linear.present(backbone):
        return None
    state = te_linear.restore_hf_layout(backbone, backbone.state_dict())
    for name, module in fused:
        prefix = name + '.'
        for key in ('gate_proj', 'up_proj', 'down_proj'):       # the inner B200MLP was un-stacked one level down
            state[prefix + key + '.weight'] = state.pop(prefix + 'mlp.' + key + '.weight')
        state[name.rsplit('.', 1)[0] + '.pre_feedforward_layernorm.weight'] = state.pop(prefix + 'layer_norm_weight')
    return state
