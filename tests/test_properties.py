"""Property tests (hypothesis) of small pure functions that everything else leans on: resize rules against the upstream
ones, visual-token selection, the compaction layout, sample selection, percentiles."""

import math

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import assume, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from prism_infer_b200.analysis import online_serving  # noqa: E402
from prism_infer_b200.analysis import quality_materialization as qmat  # noqa: E402
from prism_infer_b200.engine.kv_layout import KVLayout  # noqa: E402
from prism_infer_b200.engine.visual_pruning import target_keep_count, uniform_keep  # noqa: E402
from prism_infer_b200.engine.vl_inputs import smart_resize, smart_resize_video  # noqa: E402

FAST = settings(max_examples=300, deadline=None, derandomize=True, database=None)  # the same examples on every run


@FAST
@given(h=st.integers(32, 4000), w=st.integers(32, 4000), lo=st.sampled_from([4096, 65536, 200704]), hi=st.sampled_from([10 ** 6, 16777216]))
def test_image_resize_rule_equals_upstream_and_respects_its_budget(h, w, lo, hi):
    assume(max(h, w) / min(h, w) <= 200)
    upstream = pytest.importorskip("transformers.models.qwen2_vl.image_processing_qwen2_vl").smart_resize
    nh, nw = smart_resize(h, w, 32, lo, hi)
    assert (nh, nw) == tuple(upstream(h, w, 32, lo, hi))
    assert nh % 32 == 0 and nw % 32 == 0 and nh >= 32 and nw >= 32
    assert nh * nw <= hi


@FAST
@given(n=st.integers(1, 128), h=st.integers(32, 2000), w=st.integers(32, 2000), lo=st.sampled_from([4096, 16384, 10 ** 6]),
       hi=st.sampled_from([2 * 10 ** 6, 25165824]))
def test_clip_resize_rule_equals_upstream(n, h, w, lo, hi):
    assume(max(h, w) / min(h, w) <= 200)
    upstream = pytest.importorskip("transformers.models.qwen3_vl.video_processing_qwen3_vl").smart_resize
    assert smart_resize_video(n, h, w, 2, 32, lo, hi) == tuple(upstream(n, h, w, 2, 32, lo, hi))


@FAST
@given(n=st.integers(0, 3000), floor=st.integers(0, 1000), ratio=st.floats(0.01, 1.0))
def test_keep_count_is_bounded_and_monotone(n, floor, ratio):
    k = target_keep_count(n, floor, ratio)
    assert 0 <= k <= n and (n == 0 or k >= min(n, floor)) and (n == 0 or k >= min(n, math.ceil(n * ratio)))
    assert target_keep_count(n + 1, floor, ratio) >= k


@FAST
@given(start=st.integers(0, 500), n=st.integers(1, 600), keep=st.integers(1, 700))
def test_uniform_selection_keeps_the_ends_and_the_count(start, n, keep):
    indices = list(range(start, start + n))
    kept = uniform_keep(indices, keep)
    assert len(kept) == min(n, keep) and list(kept) == sorted(set(kept)) and set(kept) <= set(indices)
    if 2 <= keep < n:
        assert kept[0] == indices[0] and kept[-1] == indices[-1]
        gaps = [b - a for a, b in zip(kept, kept[1:])]
        assert max(gaps) - min(gaps) <= 2  # evenly spaced up to rounding


@FAST
@given(prefix=st.integers(1, 400), data=st.data())
def test_compaction_layout_maps_tail_tokens_consistently(prefix, data):
    retained = tuple(sorted(data.draw(st.sets(st.integers(0, prefix - 1), min_size=1, max_size=prefix))))
    layout = KVLayout(prefix, retained)
    assert layout.physical_prefix_len == len(retained) and layout.dropped == prefix - len(retained)
    extra = data.draw(st.integers(0, 200))
    assert layout.physical_len(prefix + extra) == len(retained) + extra
    for j in range(0, extra, max(1, extra // 5)):
        assert layout.physical_index(prefix + j) == len(retained) + j
    with pytest.raises(ValueError):
        layout.physical_index(prefix - 1)
    assert KVLayout(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in layout.record().items()}) == layout
    with pytest.raises(ValueError):
        KVLayout(prefix, retained + (prefix,))


@FAST
@given(ids=st.lists(st.integers(0, 10 ** 6), min_size=5, max_size=80, unique=True), seed=st.integers(1, 10 ** 6), data=st.data())
def test_sample_selection_is_order_independent_and_nested(ids, seed, data):
    final = data.draw(st.integers(1, len(ids)))
    dev = data.draw(st.integers(1, final))
    a = qmat.select_sample_ids(ids, dataset_id="d", revision="r", seed=seed, development_samples=dev, final_samples=final)
    b = qmat.select_sample_ids(list(reversed(ids)), dataset_id="d", revision="r", seed=seed, development_samples=dev, final_samples=final)
    assert a == b and a.final_ids[:dev] == a.development_ids and len(set(a.final_ids)) == final
    bigger = qmat.select_sample_ids(ids, dataset_id="d", revision="r", seed=seed, development_samples=dev, final_samples=len(ids))
    assert bigger.final_ids[:final] == a.final_ids  # a larger subset extends a smaller one


@FAST
@given(values=st.lists(st.floats(0.0, 1e6, allow_nan=False), min_size=1, max_size=60), q1=st.floats(0.0, 1.0), q2=st.floats(0.0, 1.0))
def test_percentiles_are_monotone_and_inside_the_data(values, q1, q2):
    lo, hi = sorted((q1, q2))
    a, b = online_serving.percentile(values, lo), online_serving.percentile(values, hi)
    assert min(values) - 1e-9 <= a <= b + 1e-9 <= max(values) + 2e-9
    d = online_serving.summarize_distribution(values)
    assert d["min"] <= d["p50"] <= d["p90"] <= d["p99"] <= d["max"] and d["count"] == len(values)
