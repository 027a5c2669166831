"""Host model of the W4A16 kernel's mbarrier pipeline (``rumus_b200/utils/pipeline_model.py``): the
roles' stage / parity arithmetic under random interleavings, for short and long K ranges and for
other ring depths; planted defects must be caught."""
import pytest

from rumus_b200.utils.pipeline_model import Mbar, PipelineError, run, w4a16_roles


def test_mbarrier_phase_parity_semantics():
    b = Mbar(2)
    assert b.passed(1) and not b.passed(0)        # fresh barrier: "previous" phase counts as complete
    b.arrive()
    assert not b.passed(0)
    b.arrive()
    assert b.passed(0) and not b.passed(1)        # phase 0 complete, phase 1 running
    b.arrive(); b.arrive()
    assert b.passed(1) and not b.passed(0)


@pytest.mark.parametrize("nkb", [1, 2, 3, 7, 8, 9, 16, 24, 25, 64, 172])
def test_w4a16_pipeline_runs_to_completion_under_any_schedule(nkb):
    for seed in range(25 if nkb < 64 else 4):
        assert run(w4a16_roles(nkb), seed) > 0


def test_w4a16_pipeline_other_ring_depths():
    for raw_stages, ab_stages in ((2, 1), (3, 2), (8, 3), (4, 6)):
        for seed in range(10):
            run(w4a16_roles(20, raw_stages=raw_stages, ab_stages=ab_stages), seed)


@pytest.mark.parametrize("bug,what", [("no_stage_wait", "overwritten while the MMA reads it|holds weights"),
                                      ("raw_count", "deadlock|holds k-block"),
                                      ("parity", "deadlock")])
def test_planted_defects_are_caught(bug, what):
    caught = 0
    for seed in range(20):
        try:
            run(w4a16_roles(24, bug=bug), seed)
        except PipelineError as e:
            import re
            assert re.search(what, str(e)), str(e)
            caught += 1
    assert caught >= 15


@pytest.mark.parametrize("tiles,nkb", [(1, 1), (1, 7), (2, 6), (3, 13), (5, 2)])
def test_two_cta_gemm_pair_protocol(tiles, nkb):
    from rumus_b200.utils.pipeline_model import gemm_2cta_roles
    for seed in range(12):
        assert run(gemm_2cta_roles(tiles, nkb), seed) > 0
    for stages in (2, 3):
        run(gemm_2cta_roles(tiles, nkb, stages=stages), 0)


@pytest.mark.parametrize("bug", ["peer_not_released", "half_tx"])
def test_two_cta_gemm_planted_defects_are_caught(bug):
    from rumus_b200.utils.pipeline_model import gemm_2cta_roles
    caught = 0
    for seed in range(12):
        try:
            run(gemm_2cta_roles(3, 9, bug=bug), seed)
        except PipelineError:
            caught += 1
    assert caught == 12


@pytest.mark.parametrize("rows,stages", [(1, 4), (3, 4), (4, 4), (9, 4), (23, 2), (40, 8)])
def test_norm_ring_protocol(rows, stages):
    """The bulk-copy ring of the LayerNorm backward kernel: no slot is refilled while a thread still reads
    it and every thread meets the rows in order, under random schedules."""
    from rumus_b200.utils.pipeline_model import norm_ring_roles, run
    for seed in range(20):
        assert run(norm_ring_roles(rows, stages), seed=seed) > 0


@pytest.mark.parametrize("bug", ["refill_early", "parity"])
def test_norm_ring_planted_defects_are_caught(bug):
    from rumus_b200.utils.pipeline_model import PipelineError, norm_ring_roles, run
    caught = 0
    for seed in range(40):
        try:
            run(norm_ring_roles(17, 4, bug=bug), seed=seed)
        except PipelineError:
            caught += 1
    assert caught > 0


@pytest.mark.parametrize("tiles", [0, 1, 2, 3, 8, 21])
def test_conv_stem_wgrad_protocol(tiles):
    """Window / dY double buffering and operand-tile reuse of the stem weight-gradient kernel."""
    from rumus_b200.utils.pipeline_model import conv_stem_wgrad_roles, run
    for seed in range(20):
        run(conv_stem_wgrad_roles(tiles), seed=seed)


def test_conv_stem_wgrad_needs_the_wait_for_the_previous_mmas():
    from rumus_b200.utils.pipeline_model import PipelineError, conv_stem_wgrad_roles, run
    caught = 0
    for seed in range(40):
        try:
            run(conv_stem_wgrad_roles(9, bug="no_mma_wait"), seed=seed)
        except PipelineError:
            caught += 1
    assert caught > 0
