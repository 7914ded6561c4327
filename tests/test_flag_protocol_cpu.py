"""Exhaustive check of the flag / epoch protocol behind the device barriers (host-side model, no GPU)."""

import pytest

from teletron_b200.utils.flag_protocol import Program, explore


@pytest.mark.parametrize("ranks,exchanges", [(2, 3), (3, 2)])
def test_two_barriers_per_exchange_are_safe_and_live(ranks, exchanges):
    r = explore(Program(ranks=ranks, exchanges=exchanges))
    assert r.violations == [] and r.timeouts == 0 and r.states > 100


def test_model_finds_the_overwrite_hazard_without_the_second_barrier():
    """With only the "data ready" barrier a fast rank overwrites its buffer while a slow one still reads it: the checker
    has to see that, or its silence above would mean nothing."""
    r = explore(Program(ranks=2, exchanges=2, second_barrier=False))
    assert any("read version 2" in v for v in r.violations)


def test_absent_rank_times_out_instead_of_hanging():
    r = explore(Program(ranks=3, exchanges=1, absent=2))
    assert r.violations == [] and r.timeouts > 0


def test_a_wait_that_gives_up_early_is_always_announced():
    """Any blocked wait may run out of budget while its peer is only slow.  Stale reads then exist, but never without a
    status word set somewhere, which is what the per-step check reduces over the ranks before the optimizer update."""
    r = explore(Program(ranks=2, exchanges=2, spurious_timeouts=True))
    assert r.violations == []
    quiet = explore(Program(ranks=2, exchanges=2))
    assert r.states > quiet.states
