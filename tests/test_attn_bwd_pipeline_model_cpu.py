"""Exhaustive interleaving check of the one-pass attention backward's warp-role pipeline (host-side model, no GPU)."""

import pytest

from teletron_b200.utils.pipeline_model import Variant, explore


@pytest.mark.parametrize("chunks", [1, 2, 3, 5])
def test_pipeline_has_no_hazard_and_no_deadlock(chunks):
    """Every buffer reuse of the kernel (T1, T2, the dS tile and the dO slots as staging, the two-slot rings) is ordered
    by its mbarriers in every interleaving, also when slots wrap around (five chunks reuse every slot twice)."""
    r = explore(chunks)
    assert r.violations == [] and r.states > 500


@pytest.mark.parametrize("variant,needle", [
    (Variant(wait_stage_done=False), "read dsA expecting ('stage'"),
    (Variant(release_slot_after_reduce=False), "overwrote do0 = ('stage', 0)"),
    (Variant(wait_dq_read=False), "expecting ('dQ', 0), found ('dP', 1)"),
])
def test_model_sees_each_hazard_when_its_wait_is_removed(variant, needle):
    r = explore(4, variant)
    assert any(needle in v for v in r.violations), r.violations[:5]
