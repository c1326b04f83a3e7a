"""Host-side checks of attention plans: no kernel is launched, no GPU is needed."""

import pytest
import torch

from bongard_b200 import flash_varlen, ops, packing


def test_plan_bounds_are_checked_before_any_launch():
    plan = ops.make_host_plan([5, 7], None, group=2, owners=[0, 1], state_lengths=[10, 20])
    assert (plan.own_extent, plan.state_extent) == (12, 30)
    ops.check_plan_bounds(plan, 12, 30)
    with pytest.raises(ValueError, match='state rows'):
        ops.check_plan_bounds(plan, 12, 29)
    with pytest.raises(ValueError, match='own-key rows'):
        ops.check_plan_bounds(plan, 11, 30)
    # explicit offsets: two questions on the same rows of the bank, a third further on
    plan = ops.make_host_plan([5, 7, 3], None, group=2, owners=[0, 0, 1], state_lengths=[10, 4], state_offsets=[6, 40])
    assert plan.state_extent == 44
    # a state nobody reads does not count
    assert ops.make_host_plan([5], None, group=2, owners=[0], state_lengths=[10, 99]).state_extent == 10
    for bad in (dict(owners=[0, 2], state_lengths=[1, 1]), dict(owners=[0, 1], state_lengths=[1, -1]),
                dict(owners=[0], state_lengths=[1])):
        with pytest.raises(ValueError):
            ops.make_host_plan([5, 7], None, group=2, **bad)
    with pytest.raises(ValueError):
        ops.make_host_plan([5, -1], None, group=2)


def test_prefix_bank_is_read_from_the_reference_gather():
    lengths, owners, states = [3, 4, 2], [1, 1, 0], [5, 6]
    key_lengths = [states[o] + n for o, n in zip(owners, lengths)]
    cu_k = torch.tensor([0, 9, 19, 26], dtype=torch.int32)
    total = sum(states)
    indices = torch.tensor(list(range(5, 11)) + [11, 12, 13] + list(range(5, 11)) + [14, 15, 16, 17]
                           + list(range(0, 5)) + [18, 19])
    got_owners, sizes, offsets = flash_varlen._prefix_bank(lengths, key_lengths, indices, cu_k, total)
    assert got_owners == [0, 0, 1] and sizes == [6, 5] and offsets == [5, 0]
    # no gather: private states back to back
    assert flash_varlen._prefix_bank(lengths, key_lengths, None, cu_k, total) == ([0, 1, 2], [6, 6, 5], None)
    with pytest.raises(ValueError, match='state bank holds'):
        flash_varlen._prefix_bank(lengths, key_lengths, indices, cu_k, 8)
    with pytest.raises(ValueError, match='contiguous run'):
        scrambled = indices.clone()
        scrambled[1], scrambled[2] = indices[2], indices[1]
        flash_varlen._prefix_bank(lengths, key_lengths, scrambled, cu_k, total)
    with pytest.raises(ValueError, match='at least its own keys'):
        flash_varlen._prefix_bank(lengths, [2, 9, 7], indices, cu_k, total)


def test_foreign_layouts_are_adopted():
    """A layout object that is not this package's PackedLayout but carries the reference's fields
    (bongard/packing.py:42-51) is converted once and cached on the object."""
    from types import SimpleNamespace

    positions = torch.tensor([[0, 1, 2, 0, 1, 0]])
    foreign = SimpleNamespace(positions=positions, masks={}, backend='flash',
                              cu_seqlens=torch.tensor([0, 3, 5, 6], dtype=torch.int32), key_seqlens=None,
                              key_indices=None, flash_windows=frozenset({None}), partitions={})
    assert packing.is_packed_layout(foreign)
    ours = packing.adopt_layout(foreign)
    assert ours.lengths == (3, 2, 1) and not ours.decoder and packing.adopt_layout(foreign) is ours
    # without cu_seqlens the segment starts are where the positions restart
    bare = SimpleNamespace(positions=positions, masks={}, backend='triton', cu_seqlens=None, key_seqlens=None,
                           key_indices=None, flash_windows=frozenset(), partitions={})
    assert packing.adopt_layout(bare).lengths == (3, 2, 1)
    # decoder: owners and state offsets come from the gather
    states, lengths, owners = [4, 2], [3, 2, 1], [1, 0, 1]
    indices, key_cu, off = [], [0], 0
    state_offsets = [0, 4]
    for n, o in zip(lengths, owners):
        indices += list(range(state_offsets[o], state_offsets[o] + states[o])) + list(range(6 + off, 6 + off + n))
        key_cu.append(key_cu[-1] + states[o] + n)
        off += n
    dec = SimpleNamespace(positions=positions, masks={}, backend='flash',
                          cu_seqlens=torch.tensor([0, 3, 5, 6], dtype=torch.int32),
                          key_seqlens=torch.tensor(key_cu, dtype=torch.int32), key_indices=torch.tensor(indices),
                          flash_windows=frozenset({None}), partitions={})
    ours = packing.adopt_layout(dec)
    assert ours.decoder and ours.owners == (0, 1, 0) and ours.state_lengths == (2, 4) and ours.state_offsets == (4, 0)
    assert not packing.is_packed_layout(SimpleNamespace(valid=None, positions=None, cu_seqlens=None))
    assert not packing.is_packed_layout(None)


def test_reference_packing_dispatch_binds_without_editing():
    from types import SimpleNamespace

    calls = []

    def native(lengths, windows, device, *, owners=None, state_lengths=None, backend='triton'):
        calls.append(backend)
        return 'native'

    module = SimpleNamespace(packed_layout=native)
    assert packing.serve_reference_packing(module) and packing.serve_reference_packing(module)
    assert module.packed_layout.native is native
    assert module.packed_layout([2], [None], torch.device('cpu'), backend='triton') == 'native' and calls == ['triton']
    ours = module.packed_layout([2, 3], [None], torch.device('cpu'), backend='b200')
    assert isinstance(ours, packing.PackedLayout) and ours.lengths == (2, 3)


@pytest.mark.parametrize('grid,items', [(148, 2272), (148, 148), (148, 149), (148, 5), (7, 100), (1, 9), (148, 12432)])
def test_attention_items_are_dealt_once_and_evenly(grid, items):
    """The persistent attention kernel's dealing rule (csrc/attn.cu item_index), through its host-side
    mirror: every work item goes to exactly one CTA, no CTA gets more than one item more than another, and
    over the heaviest-first list consecutive rounds run in opposite directions (the CTA that took the
    heaviest item of one round takes the lightest of the next)."""
    from bongard_b200 import _lib
    lib = _lib.load()
    ctas = min(grid, items)            # the launcher never starts more CTAs than items
    seen, per_cta = [], []
    for cta in range(ctas):
        mine, rnd = [], 0
        while True:
            it = lib.bg_attention_item_index(ctas, cta, rnd)
            assert it >= 0
            if it >= items:
                break
            mine.append(it)
            rnd += 1
        assert mine == sorted(mine)
        seen += mine
        per_cta.append(len(mine))
    assert sorted(seen) == list(range(items))
    assert max(per_cta) - min(per_cta) <= 1
    if items >= 2 * ctas:
        assert lib.bg_attention_item_index(ctas, 0, 0) == 0 and lib.bg_attention_item_index(ctas, 0, 1) == 2 * ctas - 1
    assert lib.bg_attention_item_index(ctas, ctas, 0) == -1 and lib.bg_attention_item_index(0, 0, 0) == -1
