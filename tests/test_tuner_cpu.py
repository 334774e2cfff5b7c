"""CPU suite: the parts of the tuner that need no GPU (stop rule, candidate gating, parameter ranges)."""
from alphasparse_b200 import tuner


def test_stop_rule_follows_the_reference_counters():
    # search_strategy.cc: 10 steps at the start; a better trial refills to clamp(5 * gain, 5, 25)
    s = tuner.SearchStrategy(struggle_step_num=2, clock=lambda: 0.0)
    assert s.continue_search(1.0)  # gain 1.0 -> 5 steps
    assert s.remain_step_num == 5 and s.best_gflops == 1.0
    assert s.continue_search(9.0)  # gain 8.0 -> 25 (clamped from 40)
    assert s.remain_step_num == 25
    for _ in range(25):
        assert s.continue_search(3.0)
    assert s.remain_step_num == 0 and s.struggle_step_num == 2
    assert s.continue_search(3.0) and s.continue_search(3.0)  # the two struggle steps
    assert s.continue_search() is False
    assert s.continue_search(3.0) is False


def test_stop_rule_time_limit():
    t = [0.0]
    s = tuner.SearchStrategy(struggle_step_num=100, total_allow_search_time=10.0, clock=lambda: t[0])
    assert s.continue_search(5.0)
    t[0] = 9.9
    assert s.continue_search() and s.continue_search(1.0)
    t[0] = 10.0
    assert not s.continue_search() and not s.continue_search(100.0)


def test_integer_range_is_inclusive_like_the_reference_enumerater():
    assert list(tuner.integer_range(32, 256, 32)) == [32, 64, 96, 128, 160, 192, 224, 256]
    assert list(tuner.integer_range(1, 16, 3)) == [1, 4, 7, 10, 13, 16]
    assert list(tuner.integer_range(5, 4, 1)) == []


def test_candidate_gating_on_row_statistics():
    names = lambda mn, mx, avg, srt: {c.name.split("_")[0] + "_" + c.template for c in tuner.compressed_candidates(mn, mx, avg, srt, quick=True)}
    short = names(1, 30, 5.0, False)
    assert {"S5_K3", "S1_K2", "S9_K9", "S9_K10", "S2_K6"} <= short and "S8_K7" not in short
    long_rows = names(4096, 400000, 9000.0, True)
    assert long_rows == {"S8_K7"}  # sorted strip of long rows: only the long-row template applies
    unsorted_skewed = names(0, 400000, 5.5, False)
    assert "S9_K9" in unsorted_skewed and "S5_K3" not in unsorted_skewed
    mid = names(40, 500, 120.0, True)
    assert {"S4_K4", "S6_K8", "S7_K8", "S5_K3", "S1_K2"} <= mid and "S9_K9" not in mid


def test_derive_tblock_matches_the_reference_shapes():
    assert tuner.derive_tblock("K2", 10_000, 0, 79, 128) == 79  # one CTA per BLB
    assert tuner.derive_tblock("K3", 10_000, 0, 0, 128) == 79  # ceil(TLBs / threads)
    assert tuner.derive_tblock("K4", 0, 1000, 0, 256) == 125  # 32 lanes per WLB
