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


def test_priority_policy_orders_admission_and_preemption():
    """``policy="priority"``: smaller values are admitted first (arrival order among equals); when blocks run out the
    least important running request is pre-empted, and it re-enters the queue in front of its equals."""
    from vllm_metax_b200.config import SchedulerConfig
    from vllm_metax_b200.engine.block_manager import KVCacheManager
    from vllm_metax_b200.engine.sampling_params import Request, SamplingParams
    from vllm_metax_b200.engine.scheduler import Scheduler

    def req(name, prio, t, n=6, out=14):
        r = Request(name, list(range(n)), SamplingParams(max_tokens=out, ignore_eos=True), None, arrival_time=t)
        r.priority = prio
        return r

    kv = KVCacheManager(8, 4, False)                      # 8 blocks of 4 tokens
    sch = Scheduler(SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64, policy="priority"), kv)
    for r in (req("low", 5, 0.0), req("mid-a", 1, 1.0), req("high", 0, 2.0), req("mid-b", 1, 3.0)):
        sch.add_request(r)
    assert [r.request_id for r in sch.waiting] == ["high", "mid-a", "mid-b", "low"]
    a = sch.schedule()
    assert [s.request.request_id for s in a.scheduled] == ["high", "mid-a"]     # two sequences at a time
    sch.update(a, {"high": 1, "mid-a": 1}, 0.0)
    # decode until the pool (8 blocks) is exhausted: the victim is mid-a (less important than high)
    preempted = []
    for _ in range(16):
        out = sch.schedule()
        preempted += [r.request_id for r in out.preempted]
        if preempted:
            break
        sch.update(out, {s.request.request_id: 1 for s in out.scheduled if s.samples}, 0.0)
    assert preempted == ["mid-a"]
    assert [r.request_id for r in sch.waiting][:2] == ["mid-a", "mid-b"]          # in front of its equal
    # first-come-first-served stays the default
    fcfs = Scheduler(SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64), KVCacheManager(8, 4, False))
    for r in (req("x", 5, 0.0), req("y", 0, 1.0)):
        fcfs.add_request(r)
    assert [r.request_id for r in fcfs.waiting] == ["x", "y"]
