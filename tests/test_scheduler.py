"""Scheduler behaviour that the pipelined (pipeline parallel, one step per stage in flight) engine relies on."""


def test_in_flight_requests_are_skipped_and_not_preempted():
    """Pipelined engine: requests of a launched step are neither scheduled again nor pre-empted until ``update``."""
    from vllm_metax_b200.config import SchedulerConfig
    from vllm_metax_b200.engine.block_manager import KVCacheManager
    from vllm_metax_b200.engine.sampling_params import Request, SamplingParams
    from vllm_metax_b200.engine.scheduler import Scheduler

    kv = KVCacheManager(16, 4, False)
    sch = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64), kv)
    sch.max_seqs_per_step = 2
    for i in range(4):
        sch.add_request(Request(f"r{i}", list(range(6)), SamplingParams(max_tokens=4, ignore_eos=True), None))
    a = sch.schedule()
    assert [s.request.request_id for s in a.scheduled] == ["r0", "r1"]          # per-step cap
    sch.mark_in_flight(a)
    b = sch.schedule()
    assert [s.request.request_id for s in b.scheduled] == ["r2", "r3"]          # disjoint from the step in flight
    sch.mark_in_flight(b)
    assert sch.schedule().is_empty                                             # everything is in flight
    assert sch.abort("r1")                                                     # marked only: its blocks are in use
    assert any(r.request_id == "r1" for r in sch.running)
    fin = sch.update(a, {"r0": 5, "r1": 6}, 0.0)
    assert fin == [] and all(r.request_id != "r1" for r in sch.running)
    c = sch.schedule()
    assert [s.request.request_id for s in c.scheduled] == ["r0"] and c.scheduled[0].is_decode
