"""Host-side expert cache against the reference's own cases for moe.ExpertCacheManager
(lm/moe/moe_test.go:34-59, lm/moe/routing_test.go:134-175). No GPU."""
import os

import pytest

from lib_b200 import moe
from lib_b200._capi import QmError


def test_register_evict_restore(tmp_path):
    mgr = moe.ExpertCacheManager(str(tmp_path), 4)
    weights = bytes([1, 2, 3, 4, 5, 6, 7, 8])
    mgr.register_expert(42, weights)
    mgr.evict_cold_expert(42)
    assert mgr.hot_experts() == 0
    assert os.path.exists(tmp_path / "expert_42.bin")
    assert mgr.get_expert(42) == weights
    assert mgr.hot_experts() == 1
    mgr.close()
    assert not os.path.exists(tmp_path / "expert_42.bin")      # Close removes the spilled files


def test_enforces_max_hot(tmp_path):
    mgr = moe.ExpertCacheManager(str(tmp_path), 2)
    for i in range(5):
        mgr.register_expert(i, bytes([i]))
        assert mgr.hot_experts() <= 2
    assert mgr.hot_experts() == 2
    # the two most recent registrations stayed; the rest spilled and page back in intact
    assert sorted(os.listdir(tmp_path)) == ["expert_0.bin", "expert_1.bin", "expert_2.bin"]
    for i in range(5):
        assert mgr.get_expert(i) == bytes([i])
        assert mgr.hot_experts() <= 2
    mgr.close()


def test_least_recently_used_is_the_victim(tmp_path):
    mgr = moe.ExpertCacheManager(str(tmp_path), 2)
    mgr.register_expert(0, b"a")
    mgr.register_expert(1, b"b")
    mgr.get_expert(0)                     # 0 is now the most recently used
    mgr.register_expert(2, b"c")          # spills 1, not 0
    assert sorted(os.listdir(tmp_path)) == ["expert_1.bin"]
    mgr.close()


def test_rejects_zero_max_hot_and_unknown_expert(tmp_path):
    with pytest.raises(QmError):
        moe.ExpertCacheManager(str(tmp_path), 0)
    mgr = moe.ExpertCacheManager(str(tmp_path), 1)
    with pytest.raises(QmError):
        mgr.get_expert(7)
    mgr.register_expert(3, b"")            # empty blob round-trips
    mgr.evict_cold_expert(3)
    assert mgr.get_expert(3) == b""
    mgr.close()
