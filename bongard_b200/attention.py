"""Attention modules and helpers with the reference's call surfaces.

Mirrors bongard/attention.py (project_qk, QuestionLayout, SharedMergedAttention,
install_shared_attention) and bongard/mps_inference.py (the encoder attention module and
the RMSNorm swap): modules are substituted in place, reuse the native parameter objects and
names, and accept exactly the keyword arguments the reference threads through the Hugging
Face layers (`packed_layout=`, `question_layout=`, `packed_cross=`, `bongard_encoder_windows=`).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn

from . import ops
from .packing import PackedLayout, is_packed_layout, packed_layout  # noqa: F401

_COPIED = ('config', 'layer_idx', 'layer_type', 'head_dim', 'num_key_value_groups', 'scaling',
           'attention_dropout', 'is_causal', 'attn_logit_softcapping', 'sliding_window', 'is_sliding')


def _weight(linear):
    return getattr(linear, 'weight')


def _recipe(linear):
    return getattr(linear, 'bongard_recipe', 'bf16')


def stacked_weight(module, names, attr):
    """One [sum(out), in] weight for several projections of the same input, cached on the
    module and rebuilt when a parameter object or version changes (the reference's TELinear
    stacks the same way, bongard/te_linear.py:47-55).  bf16, or an ops.Fp8Weight when the
    projections were converted to the FP8 recipe."""
    params = [_weight(getattr(module, n)) for n in names]
    fp8 = _recipe(getattr(module, names[0])) == 'fp8'
    key = (fp8,) + tuple((p.data_ptr(), p._version) for p in params)
    cached = module.__dict__.get(attr)
    if cached is None or cached[0] != key:
        w = torch.cat([p.detach().to(torch.bfloat16) for p in params]).contiguous()
        cached = (key, ops.quantize_weight(w) if fp8 else w)
        module.__dict__[attr] = cached
    return cached[1]


def _linear(x, w):
    return ops.linear_fp8(x, w) if isinstance(w, ops.Fp8Weight) else ops.linear(x, w)


def _theta(module):
    params = module.config.rope_parameters
    entry = params.get(module.layer_type, params) if isinstance(params, dict) else params
    return float(entry['rope_theta'])


def fused_qkv(module, hidden_states, *, positions=None, position_embeddings=None):
    """q, k, v as [T, heads, D] views of ONE stacked-projection output, q and k already
    RMS-normalised and rotated in place (bongard/attention.py:172-180 project_qk plus v_proj).
    Rotation angles come from `positions` (int32 [T]) when given, else from the bf16 cos/sin
    tables the rotary module produced."""
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    d = module.head_dim
    if needs_grad(module, hidden_states):
        return _fused_qkv_trainable(module, x, positions, position_embeddings)
    qkv = _linear(x, stacked_weight(module, ('q_proj', 'k_proj', 'v_proj'), '_b200_wqkv'))
    qd, kd = module.q_proj.weight.shape[0], module.k_proj.weight.shape[0]
    t = x.shape[0]
    q = qkv[:, :qd].view(t, qd // d, d)
    k = qkv[:, qd:qd + kd].view(t, kd // d, d)
    v = qkv[:, qd + kd:].view(t, kd // d, d)
    qw, kw = module.q_norm.weight.detach().to(torch.bfloat16), module.k_norm.weight.detach().to(torch.bfloat16)
    if positions is not None:
        ops.qk_norm_rope_(q, k, qw, kw, positions, ops.inv_freq(d, _theta(module), x.device), module.q_norm.eps)
    else:
        cos, sin = position_embeddings
        ops.qk_norm_rope_table_(q, k, qw, kw, cos.reshape(-1, d).to(torch.bfloat16), sin.reshape(-1, d).to(torch.bfloat16),
                                module.q_norm.eps)
    return q, k, v


def needs_grad(module, *tensors):
    """True when autograd would record this call: gradients are enabled and an input or one of the
    module's own parameters requires them.  The kernels then run through their autograd forms."""
    if not torch.is_grad_enabled():
        return False
    return any(t is not None and t.requires_grad for t in tensors) or any(p.requires_grad for p in module.parameters())


def _trainable_weight(module, names):
    """The stacked projection weight as a differentiable concatenation of the native parameters
    (the reference stacks them into one trainable parameter, bongard/te_linear.py:47-55)."""
    if any(_recipe(getattr(module, n)) == 'fp8' for n in names):
        raise ValueError('FP8 projections are forward-only; train with the bf16 recipe')
    weights = [_weight(getattr(module, n)) for n in names]
    w = weights[0] if len(weights) == 1 else torch.cat(weights)
    return w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)


def _fused_qkv_trainable(module, x, positions, position_embeddings):
    d = module.head_dim
    qkv = ops.linear_autograd(x, _trainable_weight(module, ('q_proj', 'k_proj', 'v_proj')))
    qd, kd = module.q_proj.weight.shape[0], module.k_proj.weight.shape[0]
    if positions is not None:
        return ops.qkv_norm_rope_autograd(qkv, qd // d, kd // d, d, module.q_norm.weight, module.k_norm.weight,
                                          positions=positions, freqs=ops.inv_freq(d, _theta(module), x.device),
                                          eps=module.q_norm.eps)
    cos, sin = position_embeddings
    return ops.qkv_norm_rope_autograd(qkv, qd // d, kd // d, d, module.q_norm.weight, module.k_norm.weight,
                                      cos=cos.reshape(-1, d).to(torch.bfloat16), sin=sin.reshape(-1, d).to(torch.bfloat16),
                                      eps=module.q_norm.eps)


def project_out(module, attended, hidden_shape):
    if needs_grad(module, attended):
        return ops.linear_autograd(attended, _trainable_weight(module, ('o_proj',))).view(*hidden_shape[:-1], -1)
    return _linear(attended, stacked_weight(module, ('o_proj',), '_b200_wo')).view(*hidden_shape[:-1], -1)


def as_token_major(t):
    """[1, heads, S, D] (the cache layout) or [S, heads, D] -> a [S, heads, D] view, no copy."""
    if t.ndim == 4:
        if t.shape[0] != 1:
            raise ValueError('shared state K/V must have batch size 1')
        t = t[0].transpose(0, 1)
    return t


def project_qk(module, hidden_states, position_embeddings, backend='b200'):
    """bongard/attention.py:172-180: returns q [B,Hq,L,D], k [B,Hkv,L,D], normalised and rotated."""
    q, k, _ = fused_qkv(module, hidden_states, position_embeddings=position_embeddings)
    b, l = hidden_states.shape[0], hidden_states.shape[1]
    return (q.view(b, l, -1, module.head_dim).transpose(1, 2), k.view(b, l, -1, module.head_dim).transpose(1, 2))


def qk_norm_rope(q, k, q_norm, k_norm, position_embeddings):
    """The fused surface of bongard/flash_attention.py:76-125 (metal_qk_norm_rope):
    q [B,L,Hq,D], k [B,L,Hkv,D] -> q' [B,Hq,L,D], k' [B,Hkv,L,D]."""
    b, l, hq, d = q.shape
    cos, sin = position_embeddings
    cos = cos.expand(b, l, d).reshape(-1, d).to(torch.bfloat16)
    sin = sin.expand(b, l, d).reshape(-1, d).to(torch.bfloat16)
    q2, k2 = q.reshape(b * l, hq, d), k.reshape(b * l, k.shape[2], d)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, q_norm.weight, k_norm.weight)):
        # unlike the reference's fused form (no-grad only, flash_attention.py:83-106) this one is differentiable
        q2, k2 = ops.qk_norm_rope_table_autograd(q2, k2, q_norm.weight, k_norm.weight, cos, sin, q_norm.eps)
    else:
        q2, k2 = q2.clone(), k2.clone()
        ops.qk_norm_rope_table_(q2, k2, q_norm.weight.detach().to(torch.bfloat16),
                                k_norm.weight.detach().to(torch.bfloat16), cos, sin, q_norm.eps)
    return q2.view(b, l, hq, d).transpose(1, 2), k2.view(b, l, -1, d).transpose(1, 2)


@dataclass
class QuestionLayout:
    """Same fields as bongard/attention.py:183-202: a right-padded batch of questions."""

    valid: torch.Tensor                      # bool [B, L]
    positions: torch.Tensor                  # int64 [B, L]
    masks: dict = field(default_factory=dict)
    state_groups: tuple = ()                 # ((row slice, state-bank row, state length), ...)
    backend: str = 'b200'


class B200RMSNorm(nn.Module):
    """RMSNorm with the (1 + weight) gain applied before rounding
    (bongard/mps_inference.py:70-83 MPSRMSNorm; transformers modeling_t5gemma2.py:55-69)."""

    def __init__(self, native):
        super().__init__()
        self.weight, self.eps = native.weight, native.eps

    def forward(self, x):
        if x.stride(-1) != 1:
            x = x.contiguous()
        if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
            return ops.rmsnorm_autograd(x, self.weight, self.eps)
        return ops.rmsnorm(x, self.weight.detach().to(torch.bfloat16), self.eps)


def _adopt(target, native):
    for name in _COPIED:
        setattr(target, name, getattr(native, name))
    for name, module in native.named_children():
        target.add_module(name, module)
    target.train(native.training)


class B200EncoderAttention(nn.Module):
    """Encoder self-attention (bongard/mps_inference.py:86-170 MPSEncoderAttention)."""

    def __init__(self, native):
        super().__init__()
        _adopt(self, native)

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, *,
                bongard_encoder_windows=None, packed_layout=None, **kwargs):
        from .packing import encoder_attention

        if packed_layout is not None:
            return encoder_attention(self, hidden_states, position_embeddings, packed_layout)
        b, s, _ = hidden_states.shape
        if b == 1 and not _has_padding(attention_mask):
            # One dense sequence is a pack of one segment (bongard/model.py:313-321 encode()).
            layout = _dense_layout(s, hidden_states.device, kwargs.get('position_ids'))
            return encoder_attention(self, hidden_states, position_embeddings, layout)
        # Right-padded batch (bongard/model.py:323-340 encode_batch): a token is valid iff it may
        # attend to itself; valid tokens are packed, attended and scattered back, padding rows stay zero.
        if attention_mask is None:
            valid = torch.ones(b, s, dtype=torch.bool, device=hidden_states.device)
        else:
            diag = attention_mask.diagonal(dim1=-2, dim2=-1)[:, 0]
            valid = diag if diag.dtype == torch.bool else diag == 0
        lengths = valid.sum(1).tolist()
        keep = valid.reshape(-1).nonzero().squeeze(1)
        layout = packed_layout_for(lengths, hidden_states.device)
        position_ids = kwargs.get('position_ids')
        if position_ids is not None:
            layout.positions32 = position_ids.expand(b, s).reshape(-1).index_select(0, keep).to(torch.int32)
        packed = hidden_states.reshape(b * s, -1).index_select(0, keep)
        out, _ = encoder_attention(self, packed[None], None, layout)
        full = torch.zeros(b * s, out.shape[-1], device=out.device, dtype=out.dtype)
        full.index_copy_(0, keep, out[0])
        return full.view(b, s, -1), None


def _has_padding(mask):
    if mask is None or not torch.is_tensor(mask) or mask.ndim != 4:
        return False
    diag = mask.diagonal(dim1=-2, dim2=-1)
    return bool((~diag).any()) if diag.dtype == torch.bool else bool((diag != 0).any())


def packed_layout_for(lengths, device):
    return packed_layout([n for n in lengths], [], device)


def _dense_layout(length, device, position_ids=None):
    layout = packed_layout([length], [], device)
    if position_ids is not None:
        layout.positions32 = position_ids.reshape(-1).to(torch.int32)
    return layout


class B200DecoderAttention(nn.Module):
    """Decoder merged attention over private questions and a shared state
    (bongard/attention.py:205-283 SharedMergedAttention)."""

    def __init__(self, native):
        super().__init__()
        _adopt(self, native)

    def forward(self, hidden_states, position_embeddings, merged_attention_mask=None, encoder_hidden_states=None,
                past_key_values=None, *, question_layout=None, packed_cross=None, **kwargs):
        from .packing import decoder_attention

        if is_packed_layout(question_layout):      # this module's layout or the reference's own
            return decoder_attention(self, hidden_states, position_embeddings, past_key_values, question_layout,
                                     packed_cross)
        cross = self._cross(past_key_values, encoder_hidden_states, packed_cross)
        if cross[0].stride(0) == 0:      # one shared state expanded over the batch (bongard/model.py:114-120)
            cross = (cross[0][:1], cross[1][:1])
        b, l, _ = hidden_states.shape
        if question_layout is None:
            # independent full-length rows, each reading state row min(i, rows - 1)
            valid = torch.ones(b, l, dtype=torch.bool, device=hidden_states.device)
            positions = kwargs.get('position_ids')
            positions = torch.arange(l, device=hidden_states.device).expand(b, l) if positions is None else positions.expand(b, l)
            groups = ()
        else:
            valid, positions, groups = question_layout.valid, question_layout.positions, question_layout.state_groups
        lengths = valid.sum(1).tolist()
        state_rows, s = cross[0].shape[0], cross[0].shape[2]
        if groups:
            owners = [0] * b
            state_lengths = [0] * state_rows
            for rows, index, length in groups:
                for r in range(*rows.indices(b)):
                    owners[r] = index
                state_lengths[index] = length
        else:
            owners = [min(i, state_rows - 1) for i in range(b)]
            state_lengths = [s] * state_rows
        # state bank: row r of the cache holds state r (padded to S); pack the valid parts
        ck = torch.cat([cross[0][r, :, :state_lengths[r]].transpose(0, 1) for r in range(state_rows)])
        cv = torch.cat([cross[1][r, :, :state_lengths[r]].transpose(0, 1) for r in range(state_rows)])
        keep = valid.reshape(-1).nonzero().squeeze(1)
        packed = hidden_states.reshape(b * l, -1).index_select(0, keep)
        layout = packed_layout(lengths, [], hidden_states.device, owners=owners, state_lengths=state_lengths)
        layout.positions32 = positions.reshape(-1).index_select(0, keep).to(torch.int32)
        out, _, _ = decoder_attention(self, packed[None], None, None, layout, (ck, cv))
        full = torch.zeros(b * l, out.shape[-1], device=out.device, dtype=out.dtype)
        full.index_copy_(0, keep, out[0])
        return full.view(b, l, -1), None, None

    def _cross(self, cache, encoder_hidden_states, packed_cross):
        if packed_cross is not None:
            return tuple(t if t.ndim == 4 else t.transpose(0, 1)[None] for t in packed_cross)
        if cache is not None:
            layers = cache.cross_attention_cache.layers
            if len(layers) > self.layer_idx and layers[self.layer_idx].get_seq_length() > 0:
                return layers[self.layer_idx].keys, layers[self.layer_idx].values
        # first use: project the state the way bongard/model.py:135-139 project_state_kv does
        state = encoder_hidden_states
        d = self.head_dim
        kd = self.k_proj.weight.shape[0]
        shape = (state.shape[0], state.shape[1], kd // d, d)
        if needs_grad(self, state):
            # train mode: the projection and the key norm record their backward kernels
            kv = ops.linear_autograd(state.reshape(-1, state.shape[-1]), _trainable_weight(self, ('k_proj', 'v_proj')))
            keys = ops.rmsnorm_autograd(kv[:, :kd].reshape(-1, d), self.k_norm.weight, self.k_norm.eps)
            keys = keys.view(shape).transpose(1, 2)
        else:
            kv = _linear(state.reshape(-1, state.shape[-1]), stacked_weight(self, ('k_proj', 'v_proj'), '_b200_wkv'))
            ops.qk_norm_rope_(None, kv[:, :kd].view(-1, kd // d, d), None, self.k_norm.weight.detach().to(torch.bfloat16),
                              None, None, self.k_norm.eps, rotate=False)
            keys = kv[:, :kd].view(shape).transpose(1, 2)
        values = kv[:, kd:].view(shape).transpose(1, 2)
        if cache is not None:
            cache.cross_attention_cache.update(keys, values, self.layer_idx)
        return keys, values


def install_shared_attention(backbone):
    """bongard/attention.py:286-289 with the B200 module."""
    for layer in backbone.decoder.layers:
        if not isinstance(layer.self_attn, B200DecoderAttention):
            layer.self_attn = B200DecoderAttention(layer.self_attn)
