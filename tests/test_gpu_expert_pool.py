"""Device-side expert residency (qm_expert_pool_*) over the host cache: least-recently-used replacement with the
policy of the reference's host cache (lm/moe/moe.go:229-248: the expert just touched is never the victim), and
every expert handed out multiplies like a freshly uploaded copy, also after a round trip through the host
cache's spill file."""
import numpy as np
import pytest

import lib_b200
from lib_b200 import moe, synth

pytestmark = pytest.mark.gpu


def test_pool_pages_experts_in_lru_order(ctx, tmp_path):
    fmt, rows, cols, experts = 12, 64, 512, 6
    blobs = [synth.weights(fmt, rows, cols, 300 + e) for e in range(experts)]
    cache = moe.ExpertCacheManager(str(tmp_path), 2)          # host memory holds two, the rest live in files
    for e, b in enumerate(blobs):
        cache.register_expert(e, b)
    pool = moe.ExpertPool(ctx, cache, fmt, rows, cols, 3)
    x = synth.activations(2, cols, 9)

    def check(e):
        w = pool.get(e)
        ref = ctx.store_upload(fmt, rows, cols, blobs[e])
        assert np.array_equal(ctx.matvec_host(w, x), ctx.matvec_host(ref, x))
        ref.free()

    for e in (0, 1, 2):
        check(e)
    assert pool.info() == (3, 3, 0, 3)
    check(1)                                   # a hit: nothing is copied
    assert pool.info() == (3, 3, 1, 3)
    check(3)                                   # replaces expert 0, the least recently used
    check(1)
    check(2)
    assert pool.info() == (3, 3, 3, 4)
    check(0)                                   # expert 0 comes back over expert 3, from the host cache's file
    check(1)
    check(2)
    assert pool.info() == (3, 3, 5, 5)
    pool.evict(2)
    assert pool.info()[0] == 2
    check(5)                                   # takes the entry that was freed: 0 and 1 stay
    check(0)
    check(1)
    assert pool.info() == (3, 3, 7, 6)
    with pytest.raises(lib_b200.QmError) as err:
        pool.get(17)                           # the host cache does not know it
    assert err.value.code == -5
    pool.close()
    cache.close()


def test_pool_refusals(ctx, tmp_path):
    cache = moe.ExpertCacheManager(str(tmp_path), 2)
    with pytest.raises(lib_b200.QmError):
        moe.ExpertPool(ctx, cache, 12, 64, 512, 0)            # "maxHot must be positive"
    with pytest.raises(lib_b200.QmError):
        moe.ExpertPool(ctx, cache, 12, 64, 500, 2)            # not a whole number of blocks
    cache.register_expert(0, synth.weights(12, 32, 512, 1))   # a blob of another shape than the pool's
    pool = moe.ExpertPool(ctx, cache, 12, 64, 512, 2)
    with pytest.raises(lib_b200.QmError) as err:
        pool.get(0)
    assert err.value.code == -2
    pool.close()
    cache.close()
