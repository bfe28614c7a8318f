"""The allocation-free decode entry point, called through its exported C symbol.

Some users of this library run under a fixed memory plan (buffers sized once at start-up, or a
host allocator they do not own) and cannot give the split-KV decode kernel a workspace.  For
them `b200_paged_decode_noalloc` keeps the workspace in a static device array inside the
library.  This file calls it the way such a user would - ctypes on the shared object, raw
pointers, no torch op - and checks it against the regular op on two calls in a row, since the
built-in workspace is shared and keeps the previous call's contents.

Collected last on purpose (file name), so a failure here cannot hide other tests behind `-x`.
"""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parents[1] / "vllm_metax_b200" / "_b200_C.so"
SCRATCH_FLOATS = 4 << 20


def _load():
    from vllm_metax_b200 import _custom_ops as ops

    assert ops.load_native(), "native library not built"
    lib = ctypes.CDLL(str(LIB))
    fn = lib.b200_paged_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 6 + [ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                                                ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200_noalloc_last_error.restype = ctypes.c_char_p
    # set-up call (first on the device): symbol address, shared-memory limit, driver-side module load
    q, cache, bt, sl = _case(99, [20, 40])
    assert _raw(fn, torch.empty_like(q), q, cache, bt, sl, 2) == 0
    torch.cuda.synchronize()
    return ops, lib, fn


def _case(seed, lens, Hq=32, Hkv=8, D=128, bs=16):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + 2
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o:o + nblk[b]].to(torch.int32)
        o += nblk[b]
    cache = torch.randn(total, 2, bs, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16).cuda()
    return q, cache, bt.cuda(), torch.tensor(lens, dtype=torch.int32).cuda()


def _call(fn, q, cache, bt, sl, splits):
    out = torch.empty_like(q)
    B, Hq, D = q.shape
    torch.cuda.synchronize()
    n_alloc = torch.cuda.memory_stats()["allocation.all.allocated"]
    free_before = torch.cuda.mem_get_info()[0]
    rc = _raw(fn, out, q, cache, bt, sl, splits)
    torch.cuda.synchronize()
    # the call allocated nothing: neither through torch's caching allocator nor behind its back (driver view).
    # The very first use of the library on a device makes the driver load its kernels and the 16 MiB array
    # (lazy module loading) - that one-time set-up is done by the warm-up call in _load().
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == n_alloc
    assert torch.cuda.mem_get_info()[0] >= free_before
    return rc, out


def _raw(fn, out, q, cache, bt, sl, splits):
    B, Hq, D = q.shape
    return fn(out.data_ptr(), q.data_ptr(), cache.data_ptr(), None, bt.data_ptr(), sl.data_ptr(), B, Hq,
            cache.shape[3], D, cache.shape[2], bt.shape[1], cache.shape[0], splits, D ** -0.5, 0, 0,
            torch.cuda.current_stream().cuda_stream)


def test_noalloc_decode_matches_regular_op_twice():
    ops, lib, fn = _load()
    # two different problems back to back: the second must not be affected by what the first
    # left in the shared workspace (more splits and longer rows first, fewer afterwards)
    for seed, lens, splits in ((0, [700, 33, 1025, 250, 1], 4), (1, [90, 512, 17], 2)):
        q, cache, bt, sl = _case(seed, lens)
        rc, got = _call(fn, q, cache, bt, sl, splits)
        assert rc == 0, lib.b200_noalloc_last_error().decode()
        torch.cuda.synchronize()
        want = ops.paged_attention_decode(q, cache, bt, sl, q.shape[-1] ** -0.5, num_splits=splits)
        torch.cuda.synchronize()
        a, b = got.float().flatten(), want.float().flatten()
        assert 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm())) < 2e-4
        torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)
        # and against the fp32 PyTorch statement of paged attention, not only against the same kernel
        from vllm_metax_b200.ops import reference as ref

        qsl = torch.arange(len(lens) + 1, dtype=torch.int32, device="cuda")
        oracle = ref.paged_attention(q, cache, bt, sl, qsl, q.shape[-1] ** -0.5)
        torch.testing.assert_close(got.float(), oracle.float(), rtol=3e-2, atol=3e-2)


def test_noalloc_decode_rejects_oversized_request():
    ops, lib, fn = _load()
    q, cache, bt, sl = _case(2, [40] * 4)
    B, Hq, D = q.shape
    splits = SCRATCH_FLOATS // (B * Hq * (D + 1)) + 1
    rc, _ = _call(fn, q, cache, bt, sl, splits)
    assert rc < 0
    assert b"scratch" in lib.b200_noalloc_last_error()
    # and the entry point still works afterwards
    rc, got = _call(fn, q, cache, bt, sl, 2)
    assert rc == 0
    want = ops.paged_attention_decode(q, cache, bt, sl, D ** -0.5, num_splits=2)
    torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)


def test_noalloc_decode_rejects_bad_sizes_before_launching():
    """Sizes an embedder could get wrong are refused with a negative code; nothing is launched for them."""
    ops, lib, fn = _load()
    q, cache, bt, sl = _case(3, [40] * 2)
    out = torch.empty_like(q)
    B, Hq, D = q.shape
    good = dict(batch=B, hq=Hq, hkv=cache.shape[3], d=D, bs=cache.shape[2], mb=bt.shape[1], nb=cache.shape[0])

    def call(**over):
        a = dict(good, **over)
        return fn(out.data_ptr(), q.data_ptr(), cache.data_ptr(), None, bt.data_ptr(), sl.data_ptr(), a["batch"], a["hq"],
                  a["hkv"], a["d"], a["bs"], a["mb"], a["nb"], 2, D ** -0.5, 0, 0, torch.cuda.current_stream().cuda_stream)

    for bad in (dict(bs=0), dict(bs=-16), dict(bs=24), dict(mb=0), dict(nb=0), dict(hq=0), dict(hkv=0), dict(d=96),
                dict(d=0), dict(batch=-1), dict(hq=Hq + 1)):
        assert call(**bad) < 0, bad
        assert lib.b200_noalloc_last_error() != b""
    assert call() == 0
    torch.cuda.synchronize()
    ops.check_kernel_status(0)
