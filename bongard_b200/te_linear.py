"""Stacked projections and the gated MLP with the reference's te_linear call surface.

Mirrors bongard/te_linear.py: `enable_te_linear(model, *, mlp=None, attention=None)` converts
every text layer's MLP and / or attention projections and returns converted-module counts;
`B200Linear` serves one or more stacked Hugging Face linears of the same input with ONE GEMM
(the reference's TELinear, 41-77), `B200MLP` runs gate_up -> GeGLU -> down as two GEMMs
(the reference's TEMLP, 79-103) with the activation fused into the first GEMM's epilogue.
Recipes here: 'bf16' (what the reference serves in eval mode, 61-62), 'fp8' (E4M3 with dynamic
per-128 block scales) and 'mxfp8' (E4M3 with power-of-two scales per 32 elements, scaled inside the
tensor core - the reference's recipe of the same name, 32-39).  Unlike the reference's modules these run the low-precision
recipe in eval mode too: that is the point of an inference kernel library.
"""

from __future__ import annotations

from collections import Counter

import torch
from torch import nn

from . import ops

RECIPES = ('bf16', 'fp8', 'mxfp8')
ATTENTION_PROJECTIONS = ('q_proj', 'k_proj', 'v_proj', 'o_proj')


class B200Linear(nn.Module):
    """y = x W^T for W = cat(linear.weight for linear in linears); `splits` are the original widths."""

    def __init__(self, linears, recipe='bf16'):
        super().__init__()
        if recipe not in RECIPES:
            raise ValueError(f'recipe must be one of {RECIPES}')
        if any(linear.bias is not None for linear in linears):
            raise ValueError('B200 projections require bias-free linears')
        self.bongard_recipe = recipe
        self.splits = [linear.out_features for linear in linears]
        self.in_features, self.out_features, self.bias = linears[0].in_features, sum(self.splits), None
        if len(linears) == 1:
            self.weight = linears[0].weight          # the native parameter object: state_dict keys stay HF-shaped
        else:
            # stacked rows as one parameter, trainable when its sources are (bongard/te_linear.py:47-55)
            self.weight = nn.Parameter(torch.cat([linear.weight.detach() for linear in linears], 0),
                                       requires_grad=all(linear.weight.requires_grad for linear in linears))
        self._cache = None
        self.counts = Counter()

    def _operand(self):
        key = (self.weight.data_ptr(), self.weight._version)
        if self._cache is None or self._cache[0] != key:
            w = self.weight.detach().to(torch.bfloat16).contiguous()
            prepare = {'bf16': lambda t: t, 'fp8': ops.quantize_weight, 'mxfp8': ops.quantize_mxfp8}[self.bongard_recipe]
            self._cache = (key, prepare(w))
            self.counts['weight_preparations'] += 1
        return self._cache[1]

    def forward(self, x, *, geglu=False):
        if self.training and torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
            # train mode: the reference goes through autograd here (bongard/te_linear.py:63-77); the bf16
            # recipe records a tensor-core backward, the fp8 recipe is an inference recipe
            if self.bongard_recipe != 'bf16':
                raise ValueError(f"the '{self.bongard_recipe}' recipe is forward-only; train with recipe 'bf16'")
            w = self.weight if self.weight.dtype == torch.bfloat16 else self.weight.to(torch.bfloat16)
            return ops.linear_geglu_autograd(x, w) if geglu else ops.linear_autograd(x, w)
        w = self._operand()
        if self.bongard_recipe == 'fp8':
            return ops.linear_fp8(x, w, geglu=geglu)
        if self.bongard_recipe == 'mxfp8':
            return ops.linear_mxfp8(x, w, geglu=geglu)
        return ops.linear_geglu(x, w) if geglu else ops.linear(x, w)


class B200MLP(nn.Module):
    """down(gelu_tanh(gate x) * up x) as a GEMM with GeGLU epilogue plus a GEMM
    (transformers modeling_t5gemma2.py:87-91; bongard/te_linear.py:98-103)."""

    def __init__(self, mlp, recipe='bf16'):
        super().__init__()
        if mlp.config.hidden_activation != 'gelu_pytorch_tanh' or mlp.dropout.p:
            raise ValueError('B200 MLP requires tanh GELU and zero dropout')
        self.bongard_recipe = recipe
        self.intermediate_size = mlp.intermediate_size
        self.fused_gate_up = True
        self.gate_up = B200Linear([mlp.gate_proj, mlp.up_proj], recipe)
        self.down = B200Linear([mlp.down_proj], recipe)

    def forward(self, x):
        if self.bongard_recipe == 'mxfp8' and not (self.training and torch.is_grad_enabled() and x.requires_grad):
            # the hidden activation goes from the GeGLU epilogue to the down projection as MXFP8
            return ops.mlp_mxfp8(x, self.gate_up._operand(), self.down._operand())
        return self.down(self.gate_up(x, geglu=True))


def _layers(model):
    backbone = model.backbone if hasattr(model, 'backbone') else model
    return list(backbone.encoder.text_model.layers) + list(backbone.decoder.layers)


def enable_te_linear(model, *, mlp=None, attention=None):
    """Convert MLP projections and/or attention projections of every text layer
    (bongard/te_linear.py:108-137).  Returns {'mlp': n, 'attention': n}."""
    if not (mlp or attention):
        raise ValueError('B200 projections require at least one recipe')
    for recipe in (mlp, attention):
        if recipe is not None and recipe not in RECIPES:
            raise ValueError(f'recipe must be one of {RECIPES}')
    ops.device_check()
    counts = Counter()
    for layer in _layers(model):
        if mlp:
            if isinstance(layer.mlp, B200MLP):
                if layer.mlp.bongard_recipe != mlp:
                    raise ValueError('An existing B200 MLP must retain its recipe')
            else:
                layer.mlp = B200MLP(layer.mlp, mlp)
            counts['mlp'] += 1
        if attention:
            for name in ATTENTION_PROJECTIONS:
                module = getattr(layer.self_attn, name)
                if isinstance(module, B200Linear):
                    if module.bongard_recipe != attention:
                        raise ValueError('An existing B200 projection must retain its recipe')
                else:
                    setattr(layer.self_attn, name, B200Linear([module], attention))
                counts['attention'] += 1
    return dict(counts)


def present(backbone):
    return any(isinstance(m, (B200Linear, B200MLP)) for m in backbone.modules())


def restore_hf_layout(backbone, state):
    """Rename the converted projections' weights in `state` (a state_dict of `backbone`) to the Hugging
    Face module keys (bongard/te_linear.py:144-161): `mlp.gate_up.weight` is split into `mlp.gate_proj.weight`
    and `mlp.up_proj.weight`, `mlp.down.weight` becomes `mlp.down_proj.weight`; converted attention
    projections already carry their native keys.  Returns `state`."""
    for name, module in backbone.named_modules():
        if isinstance(module, B200MLP):
            prefix = name + '.'
            gate, up = state.pop(prefix + 'gate_up.weight').split(module.intermediate_size)
            state[prefix + 'gate_proj.weight'] = gate
            state[prefix + 'up_proj.weight'] = up
            state[prefix + 'down_proj.weight'] = state.pop(prefix + 'down.weight')
    return state
