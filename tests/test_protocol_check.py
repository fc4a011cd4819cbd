"""Model check of the epoch-flag / double-buffer protocol of the fused collective kernels (all interleavings, CPU)."""
import pytest

from oslo_b200.utils.protocol_check import explore


@pytest.mark.parametrize("ranks,calls", [
    (2, ["ag", "ag", "ag", "ag"]),
    (2, ["rs", "rs", "rs", "rs"]),
    (2, ["ag", "rs", "rs", "ag", "ag", "rs"]),   # the order of one transformer layer, forward then backward
    (3, ["ag", "rs", "ag"]),
    (3, ["rs", "rs", "rs"]),
])
def test_double_buffered_protocol_is_safe_without_trailing_barrier(ranks, calls):
    ok, states, msg = explore(ranks, calls)
    assert ok, msg
    assert states > 100  # the search really branched


def test_single_buffer_without_barrier_is_rejected():
    """Dropping the parity (one buffer, no trailing barrier) is unsafe: the checker finds the overwrite."""
    ok, _, msg = explore(2, ["ag", "ag", "ag"], double_buffered=False)
    assert not ok and ("overwrites" in msg or "finds call" in msg), msg
    ok, _, msg = explore(2, ["rs", "rs", "rs"], double_buffered=False)
    assert not ok, msg
