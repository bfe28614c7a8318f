"""Multi-GPU microbenchmarks of the fused compute + collective kernels against their NCCL + library baselines.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m vllm_metax_b200.utils.microbench_tp [--tokens 8192]

For every path the time is the max over ranks of the CUDA-event median (warm-up 3, then ``--iters`` timed launches
with a barrier before each), and the roofline time is the slower of FLOPs / measured GEMM peak and
NVLink bytes per GPU / measured link bandwidth:

* ``gemm_ar_norm``   GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather (o_proj and down_proj shapes)
                     baseline: tcgen05 GEMM + NCCL all-reduce + fused add-RMSNorm kernel
* ``ag_gemm``        all-gather -> column-parallel GEMM; baseline: NCCL all-gather + GEMM
* ``moe_a2a``        expert-parallel dispatch + combine (bf16 and fp8 on the wire) around an identity expert
                     baseline: all-gather of tokens + reduce-scatter of outputs (NCCL)
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


def roof_ms(flops: float, link_bytes: float) -> float:
    return max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="*", default=[8192, 256])
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-moe", action="store_true")
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
    fused = FusedRowParallelNorm(g, dev, max(a.tokens), H, bf)
    nw = torch.ones(H, dtype=bf, device=dev)

    for T in a.tokens:
        for name, K in (("o_proj", H // world), ("down_proj", I // world)):
            x = torch.randn(T, K, dtype=bf, device=dev)
            w = torch.randn(H, K, dtype=bf, device=dev) * 0.02
            rpr = rows_per_rank(T, world)
            shard = torch.zeros(rpr, H, dtype=bf, device=dev)
            full_res = torch.zeros(T, H, dtype=bf, device=dev)
            t_f = timed(lambda: fused(x, w, shard, nw, 1e-5, add_residual=True), a.iters, pg)

            def baseline():
                y = ops.gemm(x, w)
                dist.all_reduce(y, group=pg)
                ops.fused_add_rms_norm(y, full_res, nw, 1e-5)

            t_b = timed(baseline, a.iters, pg)
            flops = 2.0 * T * H * K
            # bytes this GPU sends: partial rows to their owners (reduce-scatter) + its normalised rows to every peer
            link = 2.0 * (T * H * 2) * (world - 1) / world
            r = roof_ms(flops, link)
            res[f"gemm_ar_norm_{name}_T{T}"] = {"fused_ms": round(t_f, 4), "nccl_baseline_ms": round(t_b, 4),
                                               "roofline_ms": round(r, 4), "of_roofline": round(r / t_f, 3),
                                               "speedup_vs_nccl": round(t_b / t_f, 2)}
        ops.check_kernel_status(dev.index or 0)

    # ---- all-gather -> GEMM (qkv-like and gate_up-like column shards)
    for T in a.tokens:
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

    # ---- expert-parallel dispatch + combine (identity experts: measures the exchange itself)
    if not a.skip_moe and world > 1:
        E, topk, Hm = 32 * world, 8, 7168
        for T in (128, 1024):
            for quant in (False, True):
                mgr = NvlinkAll2AllManager(g, T, Hm, topk, E, bf, dev, quant_fp8=quant)
                x = torch.randn(T, Hm, dtype=bf, device=dev)
                gen = torch.Generator(device="cpu").manual_seed(rank)
                ids = torch.stack([torch.randperm(E, generator=gen)[:topk] for _ in range(T)]).int().to(dev)
                wts = torch.rand(T, topk, device=dev)

                def identity(arows, a_scale, block_expert, total):
                    if a_scale is not None:
                        return arows.view(torch.float8_e4m3fn).to(bf)
                    return arows

                t_f = timed(lambda: run_experts_a2a(mgr, x, wts, ids, identity), a.iters, pg)
                allx = torch.empty(world * T, Hm, dtype=bf, device=dev)
                out = torch.empty(T, Hm, dtype=bf, device=dev)

                def baseline():
                    dist.all_gather_into_tensor(allx, x, group=pg)
                    dist.reduce_scatter_tensor(out, allx, group=pg)

                t_b = timed(baseline, a.iters, pg)
                per_dir = T * topk * Hm * (1 if quant else 2) * (world - 1) / world
                link_ms = (per_dir + T * topk * Hm * 2 * (world - 1) / world) / (LINK_GBS * 1e9) * 1e3
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
