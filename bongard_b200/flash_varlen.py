"""Packed varlen attention behind the reference's flash_varlen surface.

Mirrors bongard/flash_varlen.py: `attention(q, k, v, layout, scale, window, cross=None)` with
tensors in [1, heads, tokens, D] order.  Two differences, both extensions:
  - an ACTIVE window is accepted (the reference raises ValueError and falls back to a Triton
    kernel, bongard/flash_varlen.py:130-131);
  - the decoder path never materialises per-question copies of the state K/V
    (bongard/flash_varlen.py:61-63 `_prefix_keys`): the kernel streams the owner's state as a
    key prefix.
The custom ops keep the reference's contracts: forwards return (out shaped like q [T, Hq, D],
lse [Hq, T] fp32; bongard/flash_varlen.py:25-27, 80-82), `flash_packed_backward` returns
(dq, dk, dv) and `flash_prefix_backward` (dq, dk, dv, dck, dcv) (bongard/flash_varlen.py:30-39,
85-105), and the forwards carry the same autograd registration (bongard/flash_varlen.py:46-58,
113-126), so `attention` is differentiable: gradients come from the tensor-core backward
kernel, for active windows too.
"""

from __future__ import annotations

import torch

from . import ops


def _prefix_bank(lengths, key_lengths, indices, cu_k, state_rows):
    """Owners and state bank of a prefix call from the reference's arguments.

    The reference hands its op the whole state bank (`ck`, `cv`: one state per owner) and a gather
    `indices` over cat(bank, own keys) that lists, for every question, its owner's state rows and
    then its own rows (bongard/packing.py:86-101, bongard/flash_varlen.py:61-63).  The kernel needs
    no gather, only where each question's state starts: the first index of its key run.  Questions
    whose states start at the same row share an owner (and therefore one key stream).  An empty
    `indices` means one private state per question, back to back in question order."""
    state_lengths = [k - n for k, n in zip(key_lengths, lengths)]
    if any(s < 0 for s in state_lengths):
        raise ValueError('cu_seqlens_k must give every question at least its own keys')
    if indices is None or indices.numel() == 0:
        return list(range(len(lengths))), state_lengths, None
    if indices.numel() != sum(key_lengths):
        raise ValueError(f'indices has {indices.numel()} entries, cu_seqlens_k describes {sum(key_lengths)} keys')
    starts = indices.index_select(0, cu_k[:-1].to(torch.int64).clamp(max=indices.numel() - 1)).tolist()
    bank, owners = {}, []
    for start, state, own in zip(starts, state_lengths, lengths):
        key = (start, state) if state else (0, 0)
        if state and not 0 <= start <= state_rows - state:
            raise ValueError(f'indices address state rows {start}..{start + state}, the state bank holds {state_rows}')
        owners.append(bank.setdefault(key, len(bank)))
    offsets, sizes = [k[0] for k in bank], [k[1] for k in bank]
    # the gather must be exactly [owner's state run | own run] per question
    own_offsets = torch.tensor([state_rows + sum(lengths[:i]) for i in range(len(lengths))], device=indices.device)
    expect = []
    for i, (start, state, own) in enumerate(zip(starts, state_lengths, lengths)):
        expect.append(torch.arange(start, start + state, device=indices.device))
        expect.append(torch.arange(own, device=indices.device) + own_offsets[i])
    if not torch.equal(torch.cat(expect), indices.to(torch.int64)):
        raise ValueError('indices must list, per question, a contiguous run of state rows followed by its own rows')
    return owners, sizes, offsets


def _plan_from_cu(cu_q, window, group, device, *, decoder=False, cu_k=None, head_dim=None, backward=False,
                  indices=None, state_rows=0):
    """Attention plan from cu_seqlens tensors (synchronises: the custom-op surface carries no host lengths)."""
    lengths = (cu_q[1:] - cu_q[:-1]).tolist()
    if not decoder:
        return ops.make_plan(lengths, window, device, group=group, head_dim=head_dim, backward=backward)
    key_lengths = (cu_k[1:] - cu_k[:-1]).tolist()
    owners, state_lengths, state_offsets = _prefix_bank(lengths, key_lengths, indices, cu_k, state_rows)
    return ops.make_plan(lengths, window, device, group=group, owners=owners, state_lengths=state_lengths,
                         state_offsets=state_offsets, head_dim=head_dim, backward=backward)


def flash_packed_forward(q, k, v, cuq, cuk, scale, causal):
    """Encoder form of the op `bongard::flash_packed_forward` (bongard/flash_varlen.py:13-22):
    q [T,Hq,D], k/v [T,Hkv,D], non-causal attention inside each cu_seqlens segment."""
    if causal:
        raise ValueError('causal packed attention goes through flash_prefix_forward (state-prefix keys)')
    plan = _plan_from_cu(cuq, None, q.shape[1] // k.shape[1], q.device, head_dim=q.shape[-1])
    out, lse = ops.varlen_attention(q, k, v, plan, scale, return_lse=True)
    return out.view(q.shape), lse


def flash_prefix_forward(q, k, v, ck, cv, indices, cuq, cuk, scale):
    """Decoder form, op `bongard::flash_prefix_forward` (bongard/flash_varlen.py:66-77): keys of
    question i are [state of its owner | own_i] with bottom-right causal alignment.  `ck`, `cv` are
    the state bank and `indices` the reference's gather over cat(bank, own keys); the owners and
    state offsets are read from it and the kernel streams each state in place (nothing is
    gathered).  An empty `indices` means one state per question, back to back."""
    plan = _plan_from_cu(cuq, None, q.shape[1] // k.shape[1], q.device, decoder=True, cu_k=cuk, head_dim=q.shape[-1],
                         indices=indices, state_rows=ck.shape[0])
    out, lse = ops.varlen_attention(q, k, v, plan, scale, (ck, cv), return_lse=True)
    return out.view(q.shape), lse


def flash_packed_backward(q, k, v, cuq, cuk, out, lse, dout, scale, causal):
    """Op `bongard::flash_packed_backward` (bongard/flash_varlen.py:30-39): (dq, dk, dv)."""
    if causal:
        raise ValueError('causal packed attention goes through flash_prefix_backward (state-prefix keys)')
    plan = _plan_from_cu(cuq, None, q.shape[1] // k.shape[1], q.device, head_dim=q.shape[-1], backward=True)
    return ops.varlen_attention_backward(q, k, v, plan, scale, out, lse, dout)


def flash_prefix_backward(q, k, v, ck, cv, indices, cuq, cuk, out, lse, dout, scale):
    """Op `bongard::flash_prefix_backward` (bongard/flash_varlen.py:85-105): (dq, dk, dv, dck, dcv);
    the state gradients are written by the key-tile passes directly, so there is no gathered
    gradient to scatter back with index_add_."""
    plan = _plan_from_cu(cuq, None, q.shape[1] // k.shape[1], q.device, decoder=True, cu_k=cuk, head_dim=q.shape[-1],
                         backward=True, indices=indices, state_rows=ck.shape[0])
    return ops.varlen_attention_backward(q, k, v, plan, scale, out, lse, dout, (ck, cv))


def _register():
    """Expose the forwards and backwards as torch custom ops under the reference's names, with the
    reference's autograd registration, when that namespace is still free (the reference registers
    the same names if it is imported)."""
    try:
        packed = torch.library.custom_op('bongard::flash_packed_forward', mutates_args=())(_packed_op)
        prefix = torch.library.custom_op('bongard::flash_prefix_forward', mutates_args=())(_prefix_op)
        packed_bwd = torch.library.custom_op('bongard::flash_packed_backward', mutates_args=())(_packed_bwd_op)
        prefix_bwd = torch.library.custom_op('bongard::flash_prefix_backward', mutates_args=())(_prefix_bwd_op)
    except Exception:   # already registered by the reference package
        return False
    packed.register_fake(lambda q, k, v, cuq, cuk, scale, causal:
                         (torch.empty_like(q), q.new_empty((q.shape[1], q.shape[0]), dtype=torch.float32)))
    prefix.register_fake(lambda q, k, v, ck, cv, indices, cuq, cuk, scale:
                         (torch.empty_like(q), q.new_empty((q.shape[1], q.shape[0]), dtype=torch.float32)))
    packed_bwd.register_fake(lambda q, k, v, cuq, cuk, out, lse, dout, scale, causal:
                             (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)))
    prefix_bwd.register_fake(lambda q, k, v, ck, cv, indices, cuq, cuk, out, lse, dout, scale:
                             tuple(torch.empty_like(t) for t in (q, k, v, ck, cv)))

    def packed_context(ctx, inputs, output):
        q, k, v, cuq, cuk, ctx.scale, ctx.causal = inputs
        out, lse = output
        ctx.save_for_backward(q, k, v, cuq, cuk, out, lse)
        ctx.mark_non_differentiable(lse)

    def packed_grad(ctx, dout, ignored):
        return (*packed_bwd(*ctx.saved_tensors, dout, ctx.scale, ctx.causal), None, None, None, None)

    def prefix_context(ctx, inputs, output):
        *tensors, ctx.scale = inputs
        out, lse = output
        ctx.save_for_backward(*tensors, out, lse)
        ctx.mark_non_differentiable(lse)

    def prefix_grad(ctx, dout, ignored):
        return (*prefix_bwd(*ctx.saved_tensors, dout, ctx.scale), None, None, None, None)

    packed.register_autograd(packed_grad, setup_context=packed_context)
    prefix.register_autograd(prefix_grad, setup_context=prefix_context)
    return True


def _packed_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cuq: torch.Tensor, cuk: torch.Tensor,
                   out: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor, scale: float, causal: bool
                   ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return flash_packed_backward(q, k, v, cuq, cuk, out, lse, dout, scale, causal)


def _prefix_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ck: torch.Tensor, cv: torch.Tensor,
                   indices: torch.Tensor, cuq: torch.Tensor, cuk: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                   dout: torch.Tensor, scale: float
                   ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return flash_prefix_backward(q, k, v, ck, cv, indices, cuq, cuk, out, lse, dout, scale)


def _packed_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cuq: torch.Tensor, cuk: torch.Tensor,
               scale: float, causal: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return flash_packed_forward(q, k, v, cuq, cuk, scale, causal)


def _prefix_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ck: torch.Tensor, cv: torch.Tensor,
               indices: torch.Tensor, cuq: torch.Tensor, cuk: torch.Tensor, scale: float
               ) -> tuple[torch.Tensor, torch.Tensor]:
    return flash_prefix_forward(q, k, v, ck, cv, indices, cuq, cuk, scale)


REGISTERED = _register()


def attention(q, k, v, layout, scale, window, cross=None):
    """bongard/flash_varlen.py:129-139.  q [1,Hq,T,D], k/v [1,Hkv,T,D], cross (ck, cv) [1,Hkv,S,D];
    returns [1,Hq,T,D].  The [heads, tokens, D] storage is read in place (the kernel takes
    head and token strides), so nothing is transposed on the way in."""
    from .packing import adopt_layout

    if q.ndim != 4 or q.shape[0] != 1:
        raise ValueError('packed attention expects [1, heads, tokens, head_dim] tensors')
    layout = adopt_layout(layout)       # the reference's own PackedLayout is accepted as it is
    q3, k3, v3 = (t[0].transpose(0, 1) for t in (q, k, v))
    if k3.stride() != v3.stride():
        k3, v3 = k[0].contiguous().transpose(0, 1), v[0].contiguous().transpose(0, 1)
    cr = None
    if cross is not None:
        ck, cv = (t[0].transpose(0, 1) if t.ndim == 4 else t for t in cross)
        if ck.stride() != cv.stride():
            ck, cv = cross[0][0].contiguous().transpose(0, 1), cross[1][0].contiguous().transpose(0, 1)
        cr = (ck, cv)
    group, head_dim = q3.shape[1] // k3.shape[1], q3.shape[-1]
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q3, k3, v3) + (cr or ()))
    if needs_grad:
        out = ops.varlen_attention_autograd(q3, k3, v3, layout.plan(window, group, head_dim, backward=True), scale, cr)
    else:
        out = ops.varlen_attention(q3, k3, v3, layout.plan(window, group, head_dim), scale, cr)
    return out.view(q3.shape[0], q3.shape[1], q3.shape[2]).transpose(0, 1)[None]
