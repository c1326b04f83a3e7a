"""Packed layouts and the per-layer attention wrappers, with the reference's call surfaces.

Mirrors bongard/packing.py: `PackedLayout`, `packed_layout`, `layout_attention`,
`encoder_attention`, `decoder_attention` keep their names, argument meaning and error
behaviour, so the reference's own `forward_packed` (bongard/packing.py:228-318) and its
attention modules can call them unchanged with `backend='b200'`.  What changes is what sits
behind them: every window - active or not - is served by one CUDA kernel, so a layout never
carries dense masks, FlexAttention block masks, short/long partitions or gathered key indices.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from itertools import accumulate

import torch

from . import ops


@dataclass
class PackedLayout:
    """Same fields as the reference's PackedLayout (bongard/packing.py:42-51); `masks`,
    `key_indices` and `partitions` stay empty because the kernel needs none of them."""

    positions: torch.Tensor                      # int64 [1, T], restarting at every segment
    masks: dict = field(default_factory=dict)
    backend: str = 'b200'
    cu_seqlens: torch.Tensor | None = None       # int32 [n + 1]
    key_seqlens: torch.Tensor | None = None      # int32 [n + 1], decoder: state + own keys per question
    key_indices: torch.Tensor | None = None
    flash_windows: frozenset = frozenset()
    partitions: dict = field(default_factory=dict)
    # host-side description the attention plans are built from
    lengths: tuple = ()
    owners: tuple | None = None
    state_lengths: tuple | None = None
    positions32: torch.Tensor | None = None      # int32 [T]
    plans: dict = field(default_factory=dict)    # (window, group) -> ops.AttentionPlan
    state_offsets: tuple | None = None           # first bank row of every state (None: back to back)

    @property
    def decoder(self):
        return self.owners is not None

    def effective_window(self, window):
        """None when the window covers every segment (the reference's own test for routing a
        layer to its dense kernel, bongard/packing.py:84-85)."""
        if window is None or not self.lengths:
            return None
        reach = window if self.decoder else (window + 1) // 2
        return None if max(self.lengths) <= reach else window

    def plan(self, window, group, head_dim=None, backward=False):
        """The attention plan of a window; `backward=True` adds the key tiles of the backward passes."""
        key = (self.effective_window(window), group, head_dim, bool(backward))
        if key not in self.plans:
            self.plans[key] = ops.make_plan(self.lengths, key[0], self.positions.device, group=group,
                                            owners=self.owners, state_lengths=self.state_lengths, head_dim=head_dim,
                                            backward=backward, state_offsets=self.state_offsets)
        return self.plans[key]


def packed_layout(lengths, windows, device, *, owners=None, state_lengths=None, backend='b200'):
    """Build once per pack; every layer shares it (bongard/packing.py:54-151).

    `windows` is accepted for signature compatibility: plans are built lazily per window."""
    if backend != 'b200':
        raise ValueError(f"bongard_b200 serves backend 'b200' only, got {backend!r}")
    lengths = tuple(int(n) for n in lengths)
    if owners is not None and state_lengths is None:
        raise ValueError('decoder layouts need state_lengths')
    device = torch.device(device)
    positions = torch.cat([torch.arange(n) for n in lengths]) if lengths else torch.zeros(0, dtype=torch.long)
    cu = torch.tensor(list(accumulate(lengths, initial=0)), dtype=torch.int32)
    key_cu = None
    if owners is not None:
        key_cu = torch.tensor(list(accumulate((state_lengths[o] + n for o, n in zip(owners, lengths)), initial=0)),
                              dtype=torch.int32).to(device)
    positions = positions.to(device)
    return PackedLayout(positions[None], {}, backend, cu.to(device), key_cu, None,
                        frozenset(set(windows)), {}, lengths,
                        None if owners is None else tuple(int(o) for o in owners),
                        None if state_lengths is None else tuple(int(s) for s in state_lengths),
                        positions.to(torch.int32))


def is_packed_layout(layout):
    """True for this module's PackedLayout and for one built by the reference's own
    `packed_layout` (bongard/packing.py:42-51): both carry `positions` [1, T] and `cu_seqlens`,
    which a padded-batch QuestionLayout (`valid`, bongard/attention.py:183-202) does not."""
    return layout is not None and hasattr(layout, 'cu_seqlens') and hasattr(layout, 'positions') \
        and not hasattr(layout, 'valid')


def adopt_layout(layout):
    """A PackedLayout of this module for `layout`, which may be one the reference's own
    `packed_layout` built (bongard/packing.py:54-151).  The conversion reads the segment lengths
    from `cu_seqlens` (backend 'flash' on CUDA, packing.py:80-81) or, failing that, from the
    positions, which restart at zero at every segment (packing.py:59); a decoder layout names
    its owners through `key_seqlens` / `key_indices` (packing.py:86-101: every question's key run
    starts with its owner's state rows).  The result is cached on the foreign object, so the
    device round trip happens once per pack, not once per layer."""
    if isinstance(layout, PackedLayout):
        return layout
    cached = layout.__dict__.get('_b200_layout') if hasattr(layout, '__dict__') else None
    if cached is not None:
        return cached
    positions = layout.positions.reshape(-1)
    cu = getattr(layout, 'cu_seqlens', None)
    if cu is not None:
        bounds = cu.tolist()
    else:
        bounds = (positions == 0).nonzero().reshape(-1).tolist() + [positions.numel()]
    lengths = [b - a for a, b in zip(bounds, bounds[1:])]
    owners = state_lengths = state_offsets = None
    key_cu = getattr(layout, 'key_seqlens', None)
    if key_cu is not None:
        from .flash_varlen import _prefix_bank

        key_bounds = key_cu.tolist()
        key_lengths = [b - a for a, b in zip(key_bounds, key_bounds[1:])]
        indices = getattr(layout, 'key_indices', None)
        state_rows = int(indices.numel() and indices.max()) + 1 - sum(lengths) if indices is not None else 0
        owners, state_lengths, state_offsets = _prefix_bank(lengths, key_lengths, indices, key_cu, max(state_rows, 0))
    elif getattr(layout, 'masks', None) and any(m is not None and getattr(m, 'ndim', 4) == 4 and
                                               m.shape[-1] != m.shape[-2] for m in layout.masks.values()):
        raise ValueError("a decoder layout without key_seqlens does not say which state a question reads; build it "
                         "with backend='b200' (install_b200_inference sets model.packing_attention) or 'flash'")
    ours = PackedLayout(layout.positions, {}, 'b200', cu if cu is None else cu.to(torch.int32), key_cu, None,
                        frozenset(getattr(layout, 'flash_windows', ())), {}, tuple(lengths),
                        None if owners is None else tuple(owners),
                        None if state_lengths is None else tuple(state_lengths),
                        positions.to(torch.int32), {},
                        None if state_offsets is None else tuple(state_offsets))
    if hasattr(layout, '__dict__'):
        layout.__dict__['_b200_layout'] = ours
    return ours


def serve_reference_packing(module=None):
    """Make the reference's own `forward_packed` (bongard/packing.py:228-318) build B200 layouts.

    `forward_packed` calls `packed_layout(..., backend=model.packing_attention)` through its
    module's global name, so binding that name to a dispatcher is all it takes: backend 'b200'
    goes to this module's `packed_layout`, every other backend to the reference's own function.
    No reference source is edited.  `module` defaults to `bongard.packing` when the reference is
    importable; returns True when the name was (or already is) bound."""
    if module is None:
        import importlib
        import sys

        module = sys.modules.get('bongard.packing')
        if module is None:
            try:
                module = importlib.import_module('bongard.packing')
            except ImportError:
                return False
    native = module.packed_layout
    if getattr(native, 'b200_dispatch', False):
        return True

    def dispatch(lengths, windows, device, *, owners=None, state_lengths=None, backend='triton'):
        if backend == 'b200':
            return packed_layout(lengths, windows, device, owners=owners, state_lengths=state_lengths, backend=backend)
        return native(lengths, windows, device, owners=owners, state_lengths=state_lengths, backend=backend)

    dispatch.b200_dispatch, dispatch.native = True, native
    dispatch.__doc__ = native.__doc__
    module.packed_layout = dispatch
    return True


def layout_attention(q, k, v, layout, scale, window, cross=None, dropout=0.0):
    """bongard/packing.py:178-198.  q [1,Hq,T,D]; k, v [1,Hkv,T,D]; cross = (ck, cv) [1,Hkv,S,D]."""
    from .flash_varlen import attention

    if dropout:
        raise ValueError('Packed CUDA attention requires zero attention dropout')
    return attention(q, k, v, adopt_layout(layout), scale, window, cross)


def _project(module, hidden_states, layout_positions, position_embeddings):
    """q, k (normalised and rotated) and v as [T, heads, D] views of one projection buffer."""
    from .attention import fused_qkv

    return fused_qkv(module, hidden_states, positions=layout_positions, position_embeddings=position_embeddings)


def encoder_attention(module, hidden_states, position_embeddings, layout):
    """bongard/packing.py:201-210: projections, QK-norm + RoPE, packed attention, o_proj."""
    from .attention import needs_grad, project_out

    layout = adopt_layout(layout)
    q, k, v = _project(module, hidden_states, layout.positions32, position_embeddings)
    group = q.shape[1] // k.shape[1]
    if needs_grad(module, hidden_states):
        out = ops.varlen_attention_autograd(q, k, v, layout.plan(module.sliding_window, group, q.shape[-1], backward=True),
                                            module.scaling)
    else:
        out = ops.varlen_attention(q, k, v, layout.plan(module.sliding_window, group, q.shape[-1]), module.scaling)
    return project_out(module, out, hidden_states.shape), None


def decoder_attention(module, hidden_states, position_embeddings, cache, layout, packed_cross=None):
    """bongard/packing.py:213-225: as above with the owner's state K/V as key prefix."""
    from .attention import as_token_major, needs_grad, project_out

    layout = adopt_layout(layout)
    q, k, v = _project(module, hidden_states, layout.positions32, position_embeddings)
    if packed_cross is None:
        cross = cache.cross_attention_cache.layers[module.layer_idx]
        packed_cross = (cross.keys, cross.values)
    ck, cv = as_token_major(packed_cross[0]), as_token_major(packed_cross[1])
    group = q.shape[1] // k.shape[1]
    if needs_grad(module, hidden_states, ck, cv):
        out = ops.varlen_attention_autograd(q, k, v, layout.plan(module.sliding_window, group, q.shape[-1], backward=True),
                                            module.scaling, (ck, cv))
    else:
        out = ops.varlen_attention(q, k, v, layout.plan(module.sliding_window, group, q.shape[-1]), module.scaling, (ck, cv))
    return project_out(module, out, hidden_states.shape), None, None
