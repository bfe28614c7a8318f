"""A bounded device-side wait that runs out, on ONE GPU and without faulting or hanging anything.

The peer-store all-reduce and the reduce / norm / all-gather kernel wait for flags that another rank raises.  Here
each is launched as "rank 0 of 2" with a pointer table whose peer rows are LOCAL buffers that nothing ever writes,
and with a wait budget of a fraction of a millisecond (the budget is a launch parameter).  The wait gives up, the
kernel records {wait timeout, site, expected, observed} in the status word and returns, the host turns that into an
exception, and the context keeps working.
"""
import pytest
import torch

from vllm_metax_b200 import _custom_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
WAIT_CYCLES = 400_000          # ~0.2 ms of SM clock


def _status_after(fn) -> dict:
    import re

    ops.load_native()
    torch.cuda.synchronize()
    ops.kernel_status(0)                           # reading clears a stale word
    fn()
    torch.cuda.synchronize()                       # returns: the wait was bounded
    with pytest.raises(RuntimeError, match="wait timeout") as err:
        ops.check_kernel_status(0)
    m = re.search(r"site (\d+) \(expected (-?\d+), observed (-?\d+)\)", str(err.value))
    st = {"code": 1, "where": int(m.group(1)), "expected": int(m.group(2)), "observed": int(m.group(3))}
    # the context is still usable: an ordinary kernel runs and is correct
    a = torch.randn(64, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(128, 256, device=DEV, dtype=torch.bfloat16)
    got = ops.gemm(a, w)
    torch.cuda.synchronize()
    assert (got.float() - a.float() @ w.float().t()).abs().max() / 16 < 0.05
    ops.check_kernel_status(0)
    return st


def test_allreduce_peer_flag_never_arrives():
    tp, max_ctas, cap = 2, 160, 1 << 20
    recv = [torch.zeros(2 * tp * cap, dtype=torch.uint8, device=DEV) for _ in range(tp)]
    gather = [torch.zeros(2 * cap, dtype=torch.uint8, device=DEV) for _ in range(tp)]
    flag1 = [torch.zeros(tp * max_ctas, dtype=torch.int32, device=DEV) for _ in range(tp)]
    flag2 = [torch.zeros(tp * max_ctas, dtype=torch.int32, device=DEV) for _ in range(tp)]
    ptrs = torch.tensor([[t.data_ptr() for t in row] for row in (recv, gather, flag1, flag2)], dtype=torch.int64)
    local_sync = torch.zeros(4, dtype=torch.int32, device=DEV)
    x = torch.randn(4096, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(x)
    st = _status_after(lambda: torch.ops.b200.custom_allreduce(out, x, ptrs, tp, 0, cap, max_ctas, local_sync, 1,
                                                                WAIT_CYCLES))
    assert st["code"] == 1 and st["where"] == 150, st          # one-shot all-reduce, first flag exchange
    assert st["expected"] == 1 and st["observed"] == 0, st      # epoch 1 awaited, the peer's flag still 0


def test_reduce_norm_gather_push_flag_never_arrives():
    tp, H, T, rows_cap = 2, 1024, 8, 8
    rpr = 4
    recv = [torch.zeros(tp * rows_cap * H, dtype=torch.bfloat16, device=DEV) for _ in range(tp)]
    f1 = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(tp)]
    f2 = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(tp)]
    outb = [torch.zeros(T * H, dtype=torch.bfloat16, device=DEV) for _ in range(tp)]
    f1[0][0] = 1                                  # rank 0's own push epoch is there; rank 1's never comes
    ptrs = torch.tensor([[t.data_ptr() for t in row] for row in (recv, f1, f2, outb)], dtype=torch.int64)
    local_sync = torch.zeros(4, dtype=torch.int32, device=DEV)
    res = torch.zeros(rpr, H, dtype=torch.bfloat16, device=DEV)
    nw = torch.ones(H, dtype=torch.bfloat16, device=DEV)
    st = _status_after(lambda: torch.ops.b200.ar_norm_gather(res, nw, 1e-5, ptrs, T, H, tp, 0, rpr, rows_cap,
                                                              local_sync, True, WAIT_CYCLES))
    assert st["code"] == 1 and st["where"] in (180, 181), st
