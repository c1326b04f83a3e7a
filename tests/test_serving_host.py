"""Host-side pieces of the single-request serving path (no GPU): the encoder-state LRU with
the reference's accounting (bongard/inference.py:213-282) and fixed-size attention plans."""

import numpy as np
import torch

from bongard_b200 import ops
from bongard_b200.serving import StateCache


def key(n, tag=0):
    return tuple([tag] * n), ()


def test_state_cache_evicts_least_recently_used_by_bytes():
    state = torch.zeros(10, 8, dtype=torch.bfloat16)            # 160 bytes + 36 * 10 key bytes = 520
    cache = StateCache(3 * 520)
    for tag in range(3):
        cache.put(key(10, tag), state)
    assert cache.info()['entries'] == 3 and cache.info()['bytes'] == 3 * 520
    assert cache.get(key(10, 0)) is state                       # refreshes entry 0
    cache.put(key(10, 3), state)                                # evicts entry 1, the oldest
    assert cache.get(key(10, 1)) is None
    assert cache.get(key(10, 0)) is not None and cache.get(key(10, 2)) is not None
    info = cache.info()
    assert (info['entries'], info['bytes'], info['hits'], info['misses']) == (3, 3 * 520, 3, 1)


def test_state_cache_skips_oversize_and_disabled():
    big = torch.zeros(100, 8, dtype=torch.bfloat16)
    cache = StateCache(1000)
    cache.put(key(100), big)                                    # larger than the whole cache: not retained
    assert cache.info()['entries'] == 0
    off = StateCache(0)
    off.put(key(1), big)
    assert off.get(key(1)) is None and off.info()['entries'] == 0
    cache.put(key(2), torch.zeros(2, 8, dtype=torch.bfloat16))
    cache.clear()
    assert cache.info()['bytes'] == 0 and cache.info()['entries'] == 0


def test_padded_plan_keeps_tiles_and_rows():
    hp = ops.make_host_plan([100, 28], 64, group=2)
    pp = hp.padded(256, hp.n_tiles + 3)
    n8 = hp.n_tiles * 8
    assert np.array_equal(pp.packed[:n8], hp.packed[:n8])
    assert not pp.packed[n8:pp.n_tiles * 8].any()               # empty tiles: no rows, no keys
    lo = pp.packed[pp.n_tiles * 8:pp.n_tiles * 8 + 256]
    hi = pp.packed[pp.n_tiles * 8 + 256:]
    assert np.array_equal(lo[:128], hp.packed[n8:n8 + 128]) and np.array_equal(hi[:128], hp.packed[n8 + 128:])
    assert not lo[128:].any() and not hi[128:].any()
    assert pp.pairs == hp.pairs and pp.tokens == 256
