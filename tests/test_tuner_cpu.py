"""CPU suite: the C++ search loop driven by a model timer instead of a GPU (candidate gating,
parameter ranges, winner selection, the padding gate, the reference's stop rule)."""
import numpy as np

from alphasparse_b200 import capi, matrices as M, tuner

TEMPLATE_OF_ID = {v: k for k, v in capi.TEMPLATE.items()}


def padded_nnz(fmt, sub):
    a = fmt.arrays(sub)
    return a["val_arr"][3]


def model_timer(prefer=None, calls=None):
    """ms = padded non-zeros of the live sub-matrices (a bandwidth model), minus a bonus for `prefer`."""
    def fn(fmt, tblock, threads, reduce):
        ms = 0.0
        for i, d in enumerate(fmt.plan_descs()):
            t = TEMPLATE_OF_ID[d.template_type]
            if t == "EMPTY":
                continue
            ms += padded_nnz(fmt, i) * 1e-6 * (0.5 if t == prefer else 1.0) * (1.0 + 0.001 * (threads[i] // 128))
        if calls is not None:
            calls.append((fmt.id, tuple(threads)))
        return ms
    return fn


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


def test_candidate_parameters_follow_the_documented_grids():
    c = {x.name: x for x in tuner.compressed_candidates(1, 30, 5.0, False, quick=True)}
    assert c["S5_K3"].nodes == ["row_padding 32 1", "tlb_row"] and c["S5_K3"].launches == [(128, 1), (256, 1)]
    assert {"S9_K9_s2", "S9_K9_s5", "S9_K10_s2", "S9_K10_s5"} <= set(c)  # s in {2, hi // 2, hi}, hi = min(avg, 32) = 5
    assert c["S2_K6_m64_c1"].launches == [(128, 1), (128, 4), (256, 1), (256, 4)]
    full = {x.name for x in tuner.compressed_candidates(1, 30, 5.0, False, quick=False)}
    assert {"S1_K2_m64", "S1_K2_m192", "S3_K6_b128_c1", "S2_K6_m32_c1"} <= full
    k7 = {x.name: x for x in tuner.compressed_candidates(4096, 400000, 9000.0, True, quick=False)}
    assert list(k7) == [f"S8_K7_c{c}" for c in (128, 256, 512, 1024, 2048, 4096)]
    assert k7["S8_K7_c4096"].launches == [(256, 1), (512, 1), (1024, 1)]


def test_derive_tblock_matches_the_reference_shapes():
    assert tuner.derive_tblock("K2", 10_000, 0, 79, 128) == 79  # one CTA per BLB
    assert tuner.derive_tblock("K3", 10_000, 0, 0, 128) == 79  # ceil(TLBs / threads)
    assert tuner.derive_tblock("K4", 0, 1000, 0, 256) == 125  # 32 lanes per WLB


def test_search_picks_the_fastest_point_of_the_model():
    m, _ = M.uniform_random(2000, 12, seed=3)
    calls = []
    desc, trials, ms = tuner.search_with_timer(m, model_timer(calls=calls))
    # a pure bandwidth model prefers the graph with the least padding: the CSR5-like formats pad only the tail
    assert desc["dense"] == "dense compress" and desc["subs"][0]["template"] in ("K9", "K10") and desc["subs"][0]["threads"] == 128
    assert ms > 0 and len(trials) >= 20 and all(t.padding_rate <= tuner.PADDING_RATE_UP_BOUND for t in trials)
    assert min(t.ms for t in trials) == min(t.ms for t in trials if t.name == desc["subs"][0]["graph"])
    # every launch of one candidate is timed on the same uploaded format (one id), in sweep order
    ids = [c[0] for c in calls]
    assert len(set(ids)) < len(ids)
    desc2, _, _ = tuner.search_with_timer(m, model_timer(prefer="K6"))
    assert desc2["subs"][0]["template"] == "K6"


def test_search_divides_skewed_matrices_when_the_model_rewards_it():
    rng = np.random.default_rng(7)
    lengths = np.concatenate([rng.integers(600, 900, size=20), np.minimum(rng.zipf(2.0, size=4000), 60)])
    rng.shuffle(lengths)
    m, _ = M.from_row_lengths(lengths, 8192, seed=8)
    logs = []
    desc, trials, _ = tuner.search_with_timer(m, model_timer(prefer="K7"), log=logs.append)
    assert "rowdiv_exp" in desc["dense"] and len(desc["subs"]) > 1
    assert desc["subs"][0]["template"] == "K7"  # the strip of long rows
    assert any("whole matrix" in l for l in logs) and any(l.startswith("dense view:") for l in logs)
    assert {t.sub for t in trials} >= set(range(len(desc["subs"])))


def test_points_that_cannot_run_are_skipped():
    m, _ = M.uniform_random(1000, 8, seed=2)

    def fn(fmt, tblock, threads, reduce):
        live = [TEMPLATE_OF_ID[d.template_type] for d in fmt.plan_descs() if TEMPLATE_OF_ID[d.template_type] != "EMPTY"]
        return None if live == ["K9"] or live == ["K10"] else 1.0 + 0.01 * threads[0]

    desc, trials, _ = tuner.search_with_timer(m, fn)
    assert desc["subs"][0]["template"] not in ("K9", "K10") and all("K9" not in t.name and "K10" not in t.name for t in trials)


def test_stop_rule_ends_a_sweep_that_no_longer_improves():
    m, _ = M.uniform_random(1500, 10, seed=4)
    all_desc, all_trials, _ = tuner.search_with_timer(m, lambda f, tb, th, rd: 1.0)
    # constant time: the first trial sets the best, then 5 refill steps (gain*5 clamped to >= 5) and 0 struggle steps
    desc, trials, _ = tuner.search_with_timer(m, lambda f, tb, th, rd: 1.0, struggle_step_num=0)
    per_dense = {}
    for t in trials:
        per_dense.setdefault((t.dense, t.sub), []).append(t)
    assert all(len(v) <= 7 for v in per_dense.values()) and len(trials) < len(all_trials)
    desc3, trials3, _ = tuner.search_with_timer(m, lambda f, tb, th, rd: 1.0, struggle_step_num=3)
    assert len(trials) < len(trials3) <= len(all_trials)


def test_bandwidth_bound_pruning_skips_only_points_that_cannot_win():
    m, _ = M.uniform_random(3000, 12, seed=6)
    timer = model_timer()  # ms = padded non-zeros * 1e-6: "1 non-zero per nanosecond"
    desc, trials, ms = tuner.search_with_timer(m, timer)
    logs = []
    # 12 bytes per fp32 non-zero at the model's speed would be 12 GB/s; with an upper bound of 6 GB/s a format
    # must be smaller than half the best one to be timed at all, so that nearly everything after the first point is skipped
    d2, t2, ms2 = tuner.search_with_timer(m, timer, prune_gbs=6.0, prune_min_bytes=1, log=logs.append)
    assert len(t2) < len(trials) and any("not timed" in l for l in logs)
    # a generous bound (1000 GB/s) prunes nothing and finds the same winner
    d3, t3, ms3 = tuner.search_with_timer(m, timer, prune_gbs=1000.0, prune_min_bytes=1)
    assert len(t3) == len(trials) and d3 == desc and ms3 == ms
    # formats below the size threshold are never pruned (cache-resident kernels beat the memory bound)
    d4, t4, _ = tuner.search_with_timer(m, timer, prune_gbs=6.0)
    assert len(t4) == len(trials) and d4 == desc


def test_interrupted_search_resumes_from_its_checkpoint(tmp_path):
    """Every timed point goes to the checkpoint file at once; a second run with the same file re-times none of them
    (and one cut off half-way re-times only what is missing), and both pick the same winner."""
    m, _ = M.uniform_random(600, 8, seed=11)
    ck = str(tmp_path / "search.ckpt")
    calls = []

    def model(fmt, tb, th, rd):
        calls.append((fmt.sub_info(0).template_type, th[0], rd[0]))
        return 1.0 + 0.001 * (th[0] % 97) + 0.01 * fmt.sub_info(0).template_type

    d1, t1, ms1 = tuner.search_with_timer(m, model, quick=True, checkpoint=ck)
    n_first = len(calls)
    lines = open(ck).read().splitlines()
    assert n_first > 10 and len(lines) == len(t1)
    calls.clear()
    d2, t2, ms2 = tuner.search_with_timer(m, model, quick=True, checkpoint=ck)
    # only the final whole-matrix timings (one per dense strategy) are not checkpointed points
    assert len(calls) < n_first // 3 and d1 == d2 and abs(ms1 - ms2) < 1e-6 and len(t2) == len(t1)
    # cut the file in the middle of a line, as an interruption would
    text = open(ck).read()
    open(ck, "w").write(text[: len(text) // 2])
    calls.clear()
    d3, t3, _ = tuner.search_with_timer(m, model, quick=True, checkpoint=ck)
    assert 0 < len(calls) < n_first and d3 == d1 and len(t3) == len(t1)


def test_trial_log_is_one_json_object_per_timed_point(tmp_path):
    import json

    m, _ = M.uniform_random(2000, 12, seed=3)
    desc, trials, ms = tuner.search_with_timer(m, model_timer())
    path = str(tmp_path / "trials.jsonl")
    assert tuner.write_trials_jsonl(path, m, trials, peak_gbs=6455.6) == len(trials)
    recs = [json.loads(l) for l in open(path)]
    assert len(recs) == len(trials) and all({"graph", "threads", "ms", "gflops", "algorithmic_GBs", "roofline_frac", "padding_rate"} <= set(r) for r in recs)
    best = min(recs, key=lambda r: r["ms"])
    assert best["graph"] == desc["subs"][0]["graph"] and abs(best["ms"] - ms) <= 1e-4 * ms
    assert abs(best["gflops"] - 2.0 * m.nnz / (best["ms"] * 1e-3) * 1e-9) < 1e-6
    # appending keeps what is there
    assert tuner.write_trials_jsonl(path, m, trials[:3], append=True) == 3 and sum(1 for _ in open(path)) == len(trials) + 3
