"""Device-resident replay of a fixed-shape serving workload (benchmark helper).

``N`` requests of ``prompt_len`` tokens each generate exactly ``out_len`` tokens.  Because every
length is known up front the whole schedule is static, so all step inputs can be staged on the
device before timing starts and the decode loop can run as back-to-back CUDA-graph replays
whose last node (``advance_step``) prepares the next iteration's inputs on the device.  The
timed region therefore contains only this framework's kernels - it is the kernel-only
counterpart of ``LLM.generate`` (which also pays host scheduling and the per-step copies).
"""
from __future__ import annotations

import torch

from .. import _custom_ops as ops
from ..attention.metadata import AttentionMetadata, ForwardContext, set_forward_context


class StaticWorkload:
    def __init__(self, runner, num_seqs: int, prompt_len: int, out_len: int, prefill_tokens: int, seed: int = 0):
        self.r = runner
        self.N, self.P, self.O = num_seqs, prompt_len, out_len
        dev = runner.device
        bs = runner.block_size
        self.bps = (prompt_len + out_len + bs - 1) // bs
        assert self.bps * num_seqs <= runner.num_blocks, "KV cache too small for the static workload"
        assert num_seqs <= runner.max_seqs and self.bps <= runner.max_blocks_per_seq
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.tokens = torch.randint(0, runner.cfg.model.vocab_size, (num_seqs, prompt_len), generator=g).to(dev)
        self.block_table_all = (torch.arange(num_seqs * self.bps, dtype=torch.int32, device=dev)
                                .view(num_seqs, self.bps))
        self.seqs_per_step = max(1, prefill_tokens // prompt_len)
        self.first = torch.zeros(num_seqs, dtype=torch.int64, device=dev)
        self.token_log = torch.zeros(num_seqs, out_len, dtype=torch.int64, device=dev)
        # ---- pre-staged prefill steps
        self.prefill_steps = []
        pos = torch.arange(prompt_len, device=dev)
        for s0 in range(0, num_seqs, self.seqs_per_step):
            k = min(self.seqs_per_step, num_seqs - s0)
            T = k * prompt_len
            bt = torch.zeros(k, runner.max_blocks_per_seq, dtype=torch.int32, device=dev)
            bt[:, : self.bps] = self.block_table_all[s0:s0 + k]
            positions = pos.repeat(k)
            blk = bt[:, : self.bps].long()[:, (pos // bs)]                      # [k, P]
            slots = (blk * bs + (pos % bs)[None, :]).reshape(-1)
            qsl = (torch.arange(k + 1, device=dev, dtype=torch.int32) * prompt_len)
            md = AttentionMetadata(
                num_tokens=T, num_reqs=k, num_decodes=0, num_decode_tokens=0, query_start_loc=qsl,
                seq_lens=torch.full((k,), prompt_len, dtype=torch.int32, device=dev), block_table=bt,
                slot_mapping=slots, max_query_len=prompt_len, max_seq_len=prompt_len, block_size=bs,
                prefill_query_start_loc=qsl, max_prefill_query_len=prompt_len)
            last = (qsl[1:] - 1).long()
            self.prefill_steps.append((s0, k, self.tokens[s0:s0 + k].reshape(-1), positions, md, last))
        self.graph = None
        self.phase_events = None     # [start, prefill done, decode done] of the latest run()

    # ------------------------------------------------------------------ decode graph
    def capture(self) -> None:
        """One graph = decode forward + logits + arg-max + advance (inputs of the next step)."""
        r, N = self.r, self.N
        dev = r.device
        md = AttentionMetadata(
            num_tokens=N, num_reqs=N, num_decodes=N, num_decode_tokens=N, query_start_loc=r.query_start_loc[:N + 1],
            seq_lens=r.seq_lens[:N], block_table=r.block_table[:N], slot_mapping=r.slot_mapping[:N],
            max_query_len=1, max_seq_len=self.P + self.O, block_size=r.block_size,
            prefill_query_start_loc=r.prefill_qsl[:1], max_prefill_query_len=0)
        md.decode_num_splits = ops.decode_num_splits(N, r.model.kv_cache_spec().get("num_kv_heads", 1),
                                                     self.P + self.O, 1, r.sms)
        if md.decode_num_splits > 1:
            spec = r.model.kv_cache_spec()
            hq = r.cfg.model.num_attention_heads // max(1, r.cfg.parallel.tensor_parallel_size)
            md.decode_workspace = torch.empty(md.decode_num_splits * N * hq * (spec["head_size"] + 1),
                                              dtype=torch.float32, device=dev)
        self.decode_md = md
        self.col = torch.zeros(1, dtype=torch.int64, device=dev)
        self._reset_decode_inputs()

        def body():
            ctx = ForwardContext(md, r.kv_caches, r.positions[:N])
            with set_forward_context(ctx):
                h = r.model(r.input_ids[:N], r.positions[:N])
            logits = r.model.compute_logits(h)
            ops.argmax(logits, r.sampled[:N])
            ops.advance_step(r.input_ids, r.positions, r.seq_lens, r.slot_mapping, r.sampled, r.block_table,
                             r.block_size, N)

        stream = torch.cuda.Stream(dev)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), torch.no_grad():
            body()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        before = ops.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=stream), torch.no_grad():
            body()
        self.launches_per_replay = ops.launch_count() - before

    def _reset_decode_inputs(self) -> None:
        r, N, bs = self.r, self.N, self.r.block_size
        r.block_table[:N].zero_()
        r.block_table[:N, : self.bps] = self.block_table_all
        r.positions[:N].fill_(self.P)
        r.seq_lens[:N].fill_(self.P + 1)
        blk = self.block_table_all[:, self.P // bs].long()
        r.slot_mapping[:N] = blk * bs + self.P % bs
        r.input_ids[:N] = self.first

    def phase_ms(self) -> dict:
        """Device time of the prefill and decode parts of the latest ``run()`` (call after a synchronize)."""
        ev = self.phase_events
        if not ev:
            return {}
        return {"prefill_ms": round(ev[0].elapsed_time(ev[1]), 2), "decode_ms": round(ev[1].elapsed_time(ev[2]), 2)}

    # ------------------------------------------------------------------ correctness probe of the fused collectives
    @torch.no_grad()
    def collective_check(self) -> dict:
        """One prefill chunk and one decode step, each run twice on the same ranks and the same cache: through the
        fused NVLink path the benchmark times, and through plain GEMMs + the library all-reduce.  Returns the
        cosine distance and the largest absolute difference of the final hidden states (the two paths add the
        partial sums in different orders, in 16-bit, so they agree closely but not bit for bit)."""
        from ..parallel import state as ps

        r = self.r
        inner = getattr(r.model, "model", None)
        group = ps.get_tp_group()
        if group.world_size == 1 or inner is None:
            return {}
        saved = (getattr(inner, "fused_ar", None), getattr(group, "custom_allreduce", None))

        def fwd(ids, positions, md):
            ctx = ForwardContext(md, r.kv_caches, positions)
            with set_forward_context(ctx):
                return r.model(ids, positions).float().clone()

        counts = []
        fused_calls = []

        def both(ids, positions, md):
            from .. import _custom_ops as ops

            n0 = ops.launch_count()
            c0 = getattr(saved[0], "calls", 0)
            a = fwd(ids, positions, md)
            fused_calls.append(getattr(saved[0], "calls", 0) - c0)
            n1 = ops.launch_count()
            inner.fused_ar, group.custom_allreduce = None, None
            try:
                b = fwd(ids, positions, md)
            finally:
                inner.fused_ar, group.custom_allreduce = saved
            counts.append((n1 - n0, ops.launch_count() - n1))        # the two paths launch different kernel counts
            cos = 1.0 - float(torch.dot(a.flatten(), b.flatten()) / (a.norm() * b.norm() + 1e-12))
            return cos, float((a - b).abs().max()), float(b.abs().max())

        _, _, ids, positions, md, _ = self.prefill_steps[0]
        p_cos, p_abs, p_ref = both(ids, positions, md)
        self._reset_decode_inputs()
        N = self.N
        d_cos, d_abs, d_ref = both(r.input_ids[:N], r.positions[:N], self.decode_md)
        torch.cuda.synchronize()
        ok = p_cos < 2e-3 and d_cos < 2e-3
        return {"fused_path": bool(saved[0] is not None), "peer_allreduce": bool(saved[1] is not None),
                "multicast_gather": bool(getattr(saved[0], "out_mc", 0)),
                "nvls_reduce_max_tokens": (saved[0].nvls_max_tokens if getattr(saved[0], "nvls", None) is not None else 0),
                "prefill_tokens": int(ids.shape[0]), "cos_diff": round(max(p_cos, d_cos), 6),
                "max_abs": round(max(p_abs, d_abs), 4), "ref_max_abs": round(max(p_ref, d_ref), 3),
                "decode_cos_diff": round(d_cos, 6), "launches_fused_vs_plain": counts, "fused_calls": fused_calls, "ok": bool(ok)}

    # ------------------------------------------------------------------ the timed body
    @torch.no_grad()
    def run(self) -> int:
        """Prefill every request, then ``out_len - 1`` graph-replayed decode steps.  Returns the
        number of kernels launched."""
        r = self.r
        before = ops.launch_count()
        if self.phase_events is None and torch.cuda.is_available():
            self.phase_events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev = self.phase_events
        if ev:
            ev[0].record()
        for s0, k, ids, positions, md, last in self.prefill_steps:
            ctx = ForwardContext(md, r.kv_caches, positions)
            with set_forward_context(ctx):
                h = r.model(ids, positions)
            logits = r.model.compute_logits(h.index_select(0, last))
            ops.argmax(logits, self.first[s0:s0 + k])
        self._reset_decode_inputs()
        self.token_log[:, 0] = self.first
        launches = ops.launch_count() - before
        if ev:
            ev[1].record()
        for i in range(1, self.O):
            self.graph.replay()
            self.token_log[:, i] = r.sampled[: self.N]
        if ev:
            ev[2].record()
        return launches + (self.O - 1) * self.launches_per_replay
