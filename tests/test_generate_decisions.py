"""The generation loop's decisions, without a GPU: who starts together, when a sequence ends,
which captured step serves a batch, how keys are split."""
from llm_infer_engine_b200.engine.engine import bucket_for, kv_bucket_for
from llm_infer_engine_b200.engine.generate import finished_reason, plan_batch
from llm_infer_engine_b200.sampling import SamplingParams, uniform_for


def test_plan_batch():
    # slots limit
    assert plan_batch([10, 10, 10, 10], 6, free_slots=3, free_pages=100, page_size=64, max_seq_len=4096) == 3
    # pages limit: each needs ceil((100 + 60) / 64) = 3 pages
    assert plan_batch([100] * 5, 60, free_slots=8, free_pages=10, page_size=64, max_seq_len=4096) == 3
    # order is kept: a large request is not skipped in favour of a later small one
    assert plan_batch([10, 5000, 10], 6, free_slots=8, free_pages=10, page_size=64, max_seq_len=8192) == 1
    # generation is capped by max_seq_len when sizing
    assert plan_batch([60], 10 ** 6, free_slots=1, free_pages=1, page_size=64, max_seq_len=64) == 1
    assert plan_batch([6000], 6, free_slots=8, free_pages=10, page_size=64, max_seq_len=8192) == 0
    assert plan_batch([], 6, free_slots=8, free_pages=10, page_size=64, max_seq_len=64) == 0


def test_finished_reason():
    stop = {2, 3}
    assert finished_reason(2, 1, 10, stop, 8, 128) == "stop"            # the stop token itself is kept by the caller
    assert finished_reason(5, 8, 10, stop, 8, 128) == "length"
    assert finished_reason(5, 3, 128, stop, 8, 128) == "max_seq_len"    # main.py:274 of the reference
    assert finished_reason(5, 3, 127, stop, 8, 128) is None
    assert finished_reason(3, 8, 128, stop, 8, 128) == "stop"           # stop wins when several hold
    assert finished_reason(2, 1, 10, set(), 8, 128) is None


def test_buckets_and_runs():
    assert [bucket_for(n) for n in (1, 2, 3, 5, 8, 9, 33, 64, 65, 300)] == [1, 2, 4, 8, 8, 16, 64, 64, 128, 300]
    assert [kv_bucket_for(n, 4096) for n in (1, 512, 513, 3000, 9000)] == [512, 512, 1024, 4096, 4096]
    assert kv_bucket_for(100, 256) == 256


def test_sampling_params_and_uniforms():
    assert SamplingParams().greedy and not SamplingParams(temperature=0.7).greedy
    assert SamplingParams(top_p=1.7).top_p == 1.0 and SamplingParams(top_p=-1).top_p == 0.0     # sampler.py:12
    us = [uniform_for(7, s, c) for s in range(50) for c in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 2400
    assert abs(sum(us) / len(us) - 0.5) < 0.02
    assert uniform_for(7, 3, 4) == uniform_for(7, 3, 4) != uniform_for(8, 3, 4)
