"""CPU suite: ownership plan of the peer-memory gradient exchange (host logic only)."""
import numpy as np
import pytest

from tensotron_b200.mlp import layer_layout
from tensotron_b200.peer import MAX_SEGMENTS, ROW_BLOCK, exchange_plan


@pytest.mark.parametrize("dims", [[784, 4096, 4096, 4096, 10], [33, 17, 9], [1024, 1000, 1024, 3000, 7], [2048, 2048]])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_plan_covers_the_flat_buffer_exactly_once(dims, world):
    offs, total = layer_layout(dims)
    own_rows, owned, repl = exchange_plan(dims, world, offs)
    cover = np.zeros(total, dtype=np.int32)
    for segs in [lay for r in owned for lay in r] + repl:
        assert len(segs) <= MAX_SEGMENTS
        for off, ln in segs:
            assert off % 4 == 0 and ln % 4 == 0 and ln > 0
            cover[off:off + ln] += 1
    assert (cover == 1).all()
    for i, rows in enumerate(own_rows):
        fan_in, fan_out = dims[i], dims[i + 1]
        if rows:
            assert rows % ROW_BLOCK == 0 and rows * world >= fan_out
            # rank r owns exactly the rows [r * rows, (r + 1) * rows) of W_i
            for r in range(world):
                lo, hi = min(fan_out, r * rows), min(fan_out, (r + 1) * rows)
                assert owned[r][i] == ([(offs[i][0] + lo * fan_in, (hi - lo) * fan_in)] if hi > lo else [])
            assert repl[i][0][0] == offs[i][1]            # the bias (and the padding behind it)
        else:
            # a replicated layer is one replicated segment: weights, bias, padding
            assert all(owned[r][i] == [] for r in range(world))
            assert repl[i][0][0] == offs[i][0] and repl[i][0][1] >= fan_out * fan_in + fan_out


def test_rank_order_sum_is_what_every_rank_ends_up_with():
    """Numpy restatement of the exchange: owners sum the ranks' slots in ascending order and
    everyone receives the owner's result, so the ranks agree bit for bit."""
    dims, world = [1024, 1024, 1024, 10], 4
    offs, total = layer_layout(dims)
    _, owned_l, repl_l = exchange_plan(dims, world, offs)
    owned = [[s for lay in owned_l[r] for s in lay] for r in range(world)]
    repl = [s for lay in repl_l for s in lay]
    rng = np.random.default_rng(0)
    slots = rng.standard_normal((world, total)).astype(np.float32)    # slot s = rank s's gradients
    want = slots[0].copy()
    for s in range(1, world):
        want = want + slots[s]
    results = np.zeros((world, total), np.float32)
    for r in range(world):
        for off, ln in owned[r]:          # the owner reduces and stores to every rank
            acc = slots[0, off:off + ln].copy()
            for s in range(1, world):
                acc = acc + slots[s, off:off + ln]
            results[:, off:off + ln] = acc
        for off, ln in repl:              # everybody reduces the replicated segments itself
            acc = slots[0, off:off + ln].copy()
            for s in range(1, world):
                acc = acc + slots[s, off:off + ln]
            results[r, off:off + ln] = acc
    for r in range(world):
        assert np.array_equal(results[r], want)
