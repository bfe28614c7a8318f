"""Failure detection without touching a GPU: failures are made on the host (a forward that raises, a rank that
stops stepping) and must reach every caller as ``EngineDeadError`` (reference pattern:
tests/v1/shutdown/test_forward_error.py:21-80)."""
import os
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)


def test_forward_error_poisons_engine_and_releases_memory():
    from vllm_metax_b200 import LLM, EngineDeadError, SamplingParams

    llm = LLM(tiny_cfg(), **KW)
    eng = llm.engine
    free0 = eng.kv.num_free_blocks
    calls = {"n": 0}
    real = eng.runner._forward            # every step path (in-turn, overlapped, pipelined) runs the model through it

    def flaky(md, T):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("injected forward failure")
        return real(md, T)

    eng.runner._forward = flaky
    with pytest.raises(EngineDeadError, match="injected forward failure"):
        llm.generate([[1, 2, 3, 4, 5]] * 3, SamplingParams(max_tokens=8, ignore_eos=True))
    assert eng.dead is not None
    with pytest.raises(EngineDeadError):
        eng.add_request([1, 2, 3])
    with pytest.raises(EngineDeadError):
        eng.step()
    if free0 is not None:
        assert eng.kv.num_free_blocks == free0          # every block went back to the pool
    assert not eng.scheduler.has_unfinished()


class DictStore:
    """The three calls of a c10d store that RankLiveness uses."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_rank_liveness_protocol():
    from vllm_metax_b200.parallel.liveness import PeerFailedError, RankLiveness

    store = DictStore()
    r0, r1, r2 = (RankLiveness(store, r, 3) for r in range(3))
    r0.check()
    r1.beat(1)
    r2.beat(1)
    assert r0.stale_peers(5.0) == []
    r2.announce_failure("RuntimeError('boom')")
    with pytest.raises(PeerFailedError, match="rank 2 failed.*boom") as ei:
        r0.check()
    assert ei.value.rank == 2
    r2.check()                                    # a rank does not report itself
    store.set("b200_live/beat/1", f"7:{time.time() - 60:.3f}")
    assert r0.stale_peers(5.0) == [1]


def _rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_PG_TIMEOUT_S="6", B200_FUSED_TP_COLLECTIVES="0")
    from vllm_metax_b200 import LLM, EngineDeadError, SamplingParams

    llm = LLM(tiny_cfg(), tensor_parallel_size=world, **KW)
    eng = llm.engine
    assert eng.liveness is not None
    if rank == 1:
        def hook(when, step):
            if when == "before" and step == 2:
                raise RuntimeError("rank 1 gives up")      # between steps: nothing of this rank is in flight

        eng.step_hooks.append(hook)
    t0 = time.time()
    try:
        llm.generate([[5, 6, 7, 8]] * 2, SamplingParams(max_tokens=16, ignore_eos=True))
        q.put((rank, "finished", ""))
    except EngineDeadError as e:
        q.put((rank, "dead", str(e)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "other", repr(e)))
    assert time.time() - t0 < 60
    q.close()
    q.join_thread()      # the message must leave before the hard exit
    os._exit(0)          # the process group is broken on purpose; skip its teardown


def test_peer_failure_reaches_every_rank_as_engine_dead():
    """Rank 1 raises between two steps.  Rank 0 must end with EngineDeadError too: either its pre-step check
    sees the announcement in the store, or the collective it already entered runs into the group timeout."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + os.getpid() % 150
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        rank, state, msg = q.get(timeout=150)
        got[rank] = (state, msg)
    for p in procs:
        p.join(timeout=60)
    assert got[1][0] == "dead" and "rank 1 gives up" in got[1][1], got
    assert got[0][0] == "dead", got
