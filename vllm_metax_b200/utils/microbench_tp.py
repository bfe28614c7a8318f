"""Multi-GPU microbenchmarks of the fused compute + collective kernels against their NCCL + library baselines.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m vllm_metax_b200.utils.microbench_tp [--tokens 8192]

For every path the time is the max over ranks of the CUDA-event median (warm-up 3, then ``--iters`` timed launches
with a barrier before each), and the roofline time is the slower of FLOPs / measured GEMM peak and
NVLink bytes per GPU / measured link bandwidth:

* ``gemm_ar_norm``   GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather (o_proj and down_proj shapes)
                     baseline: tcgen05 GEMM + NCCL all-reduce + fused add-RMSNorm kernel
* ``ag_gemm``        all-gather -> column-parallel GEMM; baseline: NCCL all-gather + GEMM
* ``allreduce``      stand-alone one-shot / two-shot peer-store all-reduce against NCCL (32 KiB .. 8 MiB)
* ``reduce_rms``     cross-rank q/k RMSNorm (4-byte partial sums as their own flags) against torch ops + NCCL
* ``peer_copy``      (``--p2p``) raw bandwidth of the push primitives into the next rank's memory
* ``moe_a2a``        expert-parallel dispatch + combine (bf16 and fp8 on the wire) around an identity expert
                     baseline: all-gather of tokens / ids / weights, the same align + gather + weighted-sum kernels
                     on all tokens, reduce-scatter of the partial sums (NCCL)
Rank 0 prints one JSON object.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

GEMM_PEAK_TFLOPS = 1625.0      # measured cuBLAS bf16 burst on this pool
LINK_GBS = 770.0               # measured peer copy, per direction per GPU


def timed(fn, iters: int, group) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def graph_timed(fn, group, calls: int = 16, replays: int = 5) -> float:
    """ms per call inside a replayed CUDA graph of ``calls`` back-to-back calls (how decode steps run: no host
    launch gaps between the kernels), median over ``replays``, max over ranks."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            for _ in range(calls):
                fn()
    torch.cuda.synchronize()
    ts = []
    for i in range(replays + 2):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            ts.append(e0.elapsed_time(e1) / calls)
    t = torch.tensor([statistics.median(ts)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del g
    return float(t.item())


def roof_ms(flops: float, link_bytes: float) -> float:
    return max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="*", default=[8192, 256])
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-moe", action="store_true")
    ap.add_argument("--only", default="", help="comma list of sections: row,ag,allreduce,moe (default: all)")
    ap.add_argument("--p2p", action="store_true", help="also measure raw peer-copy bandwidth")
    a = ap.parse_args()

    from vllm_metax_b200 import _custom_ops as ops
    from vllm_metax_b200.parallel import state as ps
    from vllm_metax_b200.parallel.all2all import NvlinkAll2AllManager, run_experts_a2a
    from vllm_metax_b200.parallel.fused_collectives import AllGatherGemm, FusedRowParallelNorm, rows_per_rank

    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps.init_distributed(tensor_parallel_size=world)
    rank = ps.tp_rank()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    g = ps.get_tp_group()
    pg = g.device_pg if hasattr(g, "device_pg") else None
    H, I = a.hidden, a.inter
    res: dict = {"world": world}
    bf = torch.bfloat16
    only = set(x for x in a.only.split(",") if x)
    want = lambda sec: not only or sec in only      # noqa: E731
    fused = FusedRowParallelNorm(g, dev, max(a.tokens), H, bf)
    nw = torch.ones(H, dtype=bf, device=dev)
    res["multicast_gather"] = bool(fused.out_mc)
    res["nvls_reduce"] = fused.nvls is not None
    res["nvls_max_tokens"] = fused.nvls_max_tokens if fused.nvls is not None else 0

    for T in (a.tokens if want("row") else []):
        for name, K in (("o_proj", H // world), ("down_proj", I // world)):
            x = torch.randn(T, K, dtype=bf, device=dev)
            w = torch.randn(H, K, dtype=bf, device=dev) * 0.02
            rpr = rows_per_rank(T, world)
            shard = torch.zeros(rpr, H, dtype=bf, device=dev)
            full_res = torch.zeros(T, H, dtype=bf, device=dev)
            fused.kernel = "split"     # GEMM with row-scatter epilogue + reduce / norm / all-gather kernel
            t_f = timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), a.iters, pg)
            fused.kernel = "mono"      # the single-kernel variant
            t_m = timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), a.iters, pg)
            fused.kernel = "split"

            def baseline():
                y = ops.gemm(x, w)
                dist.all_reduce(y, group=pg)
                ops.fused_add_rms_norm(y, full_res, nw, 1e-5)

            t_b = timed(baseline, a.iters, pg)
            # the two launches of the split path on their own, and the same GEMM with an ordinary local epilogue
            t_g = timed(lambda: torch.ops.b200.gemm_row_scatter(x, w, fused.ptrs_scatter, world, rank, rpr,
                                                                 fused.rows_cap, fused.local_sync_split), a.iters, pg)
            t_n = timed(lambda: torch.ops.b200.ar_norm_gather(shard, nw, 1e-5, fused.ptrs_gather, T, H, world, rank,
                                                               rpr, fused.rows_cap, fused.local_sync_split, True,
                                                               fused.wait_cycles, fused.out_mc), a.iters, pg)
            y_loc = torch.empty(T, H, dtype=bf, device=dev)
            t_l = timed(lambda: ops.gemm(x, w, out=y_loc), a.iters, pg)
            extra = {}
            nv = fused.nvls
            if nv is not None and T <= fused.nvls_max_tokens:
                # `fused_ms` above took the in-switch reduction; the peer-store kernels at the same size:
                fused.nvls = None
                extra["peer_store_path_ms"] = round(timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), a.iters, pg), 4)
                fused.nvls = nv
            if T <= 1024:      # launch-bound sizes: per-call time inside a replayed graph
                extra["fused_in_graph_ms"] = round(graph_timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), pg), 4)
                if nv is not None:
                    fused.nvls = None
                    extra["peer_store_path_in_graph_ms"] = round(
                        graph_timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), pg), 4)
                    fused.nvls = nv
                extra["nccl_baseline_in_graph_ms"] = round(graph_timed(baseline, pg), 4)
                extra["local_gemm_in_graph_ms"] = round(graph_timed(lambda: ops.gemm(x, w, out=y_loc), pg), 4)
            flops = 2.0 * T * H * K
            # bytes this GPU sends: partial rows to their owners (reduce-scatter) + its normalised rows to every peer
            link = 2.0 * (T * H * 2) * (world - 1) / world
            r = roof_ms(flops, link)
            res[f"gemm_ar_norm_{name}_T{T}"] = {"fused_ms": round(t_f, 4), "single_kernel_ms": round(t_m, 4),
                                               "nccl_baseline_ms": round(t_b, 4), "scatter_gemm_ms": round(t_g, 4),
                                               "reduce_norm_gather_ms": round(t_n, 4), "local_gemm_ms": round(t_l, 4),
                                               "roofline_ms": round(r, 4), "of_roofline": round(r / t_f, 3),
                                               "speedup_vs_nccl": round(t_b / t_f, 2), **extra}
        ops.check_kernel_status(dev.index or 0)

    # ---- all-gather -> GEMM (qkv-like and gate_up-like column shards)
    for T in (a.tokens if want("ag") else []):
        rows = (T // world + 127) // 128 * 128
        if rows == 0:
            continue
        ag = AllGatherGemm(g, dev, rows, H, bf)
        for name, N in (("qkv", 6144 // world), ("gate_up", 2 * I // world)):
            N = (N + 7) // 8 * 8
            w = torch.randn(N, H, dtype=bf, device=dev) * 0.02
            ag.x_shard(rows).normal_()
            t_f = timed(lambda: ag(rows, w), a.iters, pg)
            xs = ag.x_shard(rows)
            gathered = torch.empty(world * rows, H, dtype=bf, device=dev)

            def baseline():
                dist.all_gather_into_tensor(gathered, xs, group=pg)
                ops.gemm(gathered, w)

            t_b = timed(baseline, a.iters, pg)
            flops = 2.0 * world * rows * N * H
            link = rows * H * 2.0 * (world - 1)                # bytes pulled in per GPU
            r = roof_ms(flops, link)
            res[f"ag_gemm_{name}_T{world * rows}"] = {"fused_ms": round(t_f, 4), "nccl_baseline_ms": round(t_b, 4),
                                                      "roofline_ms": round(r, 4), "of_roofline": round(r / t_f, 3),
                                                      "speedup_vs_nccl": round(t_b / t_f, 2)}
        ops.check_kernel_status(dev.index or 0)
        ag.close()

    # ---- stand-alone all-reduce (one-shot / two-shot peer stores) against NCCL, small to medium messages
    if world > 1 and want("allreduce"):
        from vllm_metax_b200.parallel.custom_allreduce import CrossRankRMSNorm, CustomAllReduce

        car = CustomAllReduce(g, dev, 8 << 20)
        for nbytes in (32 << 10, 512 << 10, 2 << 20, 8 << 20):
            y = torch.randn(nbytes // 2, dtype=bf, device=dev)
            t1 = timed(lambda: car.all_reduce(y, mode=1), a.iters, pg)
            t2 = timed(lambda: car.all_reduce(y, mode=2), a.iters, pg)
            tn = timed(lambda: dist.all_reduce(y, group=pg), a.iters, pg)
            link = 2.0 * nbytes * (world - 1) / world / (LINK_GBS * 1e9) * 1e3
            res[f"allreduce_{nbytes >> 10}KiB"] = {"one_shot_ms": round(t1, 4), "two_shot_ms": round(t2, 4),
                                                  "nccl_ms": round(tn, 4), "link_roofline_ms": round(link, 5)}
        ops.check_kernel_status(dev.index or 0)
        car.close()
        rms = CrossRankRMSNorm(g, dev, 8192)
        for T in (256, 8192):
            q = torch.randn(T, 6144 // world, dtype=bf, device=dev)
            k = torch.randn(T, 1024 // world if world <= 8 else 128, dtype=bf, device=dev)
            wq, wk = torch.ones(q.shape[1], dtype=bf, device=dev), torch.ones(k.shape[1], dtype=bf, device=dev)
            t_f = timed(lambda: rms(q, wq, 1e-6, k, wk), a.iters, pg)

            def baseline():
                ss = torch.stack([q.float().pow(2).sum(-1), k.float().pow(2).sum(-1)])
                dist.all_reduce(ss, group=pg)
                return (q * torch.rsqrt(ss[0] / 6144 + 1e-6)[:, None].to(bf) * wq,
                        k * torch.rsqrt(ss[1] / 1024 + 1e-6)[:, None].to(bf) * wk)

            t_b = timed(baseline, a.iters, pg)
            res[f"reduce_rms_qk_T{T}"] = {"fused_ms": round(t_f, 4), "torch_nccl_baseline_ms": round(t_b, 4)}
        ops.check_kernel_status(dev.index or 0)
        rms.close()

    # ---- raw peer-copy bandwidth of the push primitives (plain 16-byte stores, bulk stores), per CTA count
    if world > 1 and a.p2p:
        from vllm_metax_b200.parallel.symm_mem import SymmWorkspace

        n = 64 << 20
        ws = SymmWorkspace(g, n + 4096, dev)
        reg = ws.region("buf", n)
        peer = ws.peer_ptrs(reg)[(rank + 1) % world]
        src = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev)
        for mode, name in ((0, "st16"), (1, "bulk")):
            for ctas in (8, 32, 148):
                t = timed(lambda: torch.ops.b200.p2p_copy(peer, src, ctas, mode), 5, pg)
                res[f"peer_copy_{name}_ctas{ctas}_GBs"] = round(n / t / 1e6, 1)
        ops.check_kernel_status(dev.index or 0)
        ws.close()

    # ---- expert-parallel dispatch + combine (identity experts: measures the exchange itself)
    if not a.skip_moe and world > 1 and want("moe"):
        E, topk, Hm = 32 * world, 8, 7168
        for T in (128, 1024):
            for quant in (False, True):
                mgr = NvlinkAll2AllManager(g, T, Hm, topk, E, bf, dev, quant_fp8=quant)
                x = torch.randn(T, Hm, dtype=bf, device=dev)
                gen = torch.Generator(device="cpu").manual_seed(rank)
                ids = torch.stack([torch.randperm(E, generator=gen)[:topk] for _ in range(T)]).int().to(dev)
                wts = torch.rand(T, topk, device=dev)

                y_buf: dict = {}

                def identity(arows, a_scale, block_expert, total):
                    # stands for the grouped GEMMs: fp8 rows would feed the fp8 GEMM as they are, so the timing
                    # must not include a conversion - hand back a bf16 buffer of the right shape
                    if a_scale is None:
                        return arows
                    if arows.shape[0] not in y_buf:
                        y_buf[arows.shape[0]] = torch.zeros(arows.shape[0], Hm, dtype=bf, device=dev)
                    return y_buf[arows.shape[0]]

                t_f = timed(lambda: run_experts_a2a(mgr, x, wts, ids, identity), a.iters, pg)
                # baseline = the all-gather / reduce-scatter manager's path: every rank receives ALL tokens, keeps the
                # pairs of its own experts (same align / gather / weighted-sum kernels), reduce-scatters the partial sums
                allx = torch.empty(world * T, Hm, dtype=bf, device=dev)
                all_ids = torch.empty(world * T, topk, dtype=torch.int32, device=dev)
                all_w = torch.empty(world * T, topk, dtype=torch.float32, device=dev)
                out = torch.empty(T, Hm, dtype=bf, device=dev)
                el = E // world
                emap = torch.full((E,), -1, dtype=torch.int32, device=dev)
                emap[rank * el:(rank + 1) * el] = torch.arange(el, dtype=torch.int32, device=dev)

                def baseline():
                    dist.all_gather_into_tensor(allx, x, group=pg)
                    dist.all_gather_into_tensor(all_ids, ids, group=pg)
                    dist.all_gather_into_tensor(all_w, wts, group=pg)
                    sorted_ids, block_expert, total, inv = ops.moe_align_block_size(all_ids, 128, el, emap, want_inverse=True)
                    arows = ops.moe_gather(allx, sorted_ids, total, topk)
                    part = ops.moe_combine(arows, all_w, inv, world * T, None)
                    dist.reduce_scatter_tensor(out, part, group=pg)

                t_b = timed(baseline, a.iters, pg)
                # rows that really cross NVLink: one per (token, remote rank owning one of its experts), both ways
                dst = ids // el
                remote = sum(int(((dst == r).any(dim=1)).sum()) for r in range(world) if r != rank)
                link_ms = remote * Hm * ((1 if quant else 2) + 2) / (LINK_GBS * 1e9) * 1e3
                res[f"moe_a2a_T{T}_{'fp8' if quant else 'bf16'}"] = {
                    "fused_ms": round(t_f, 4), "nccl_agrs_baseline_ms": round(t_b, 4), "link_roofline_ms": round(link_ms, 4),
                    "of_roofline": round(link_ms / t_f, 3), "speedup_vs_nccl": round(t_b / t_f, 2)}
                ops.check_kernel_status(dev.index or 0)
                mgr.close()
    if rank == 0:
        print(json.dumps(res, indent=1))
    torch.cuda.synchronize()
    import threading

    threading.Timer(20.0, lambda: os._exit(0)).start()
    ps.destroy()
    os._exit(0)


if __name__ == "__main__":
    main()
