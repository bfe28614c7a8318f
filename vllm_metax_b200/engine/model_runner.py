"""Executes one scheduler step on this rank's GPU.

Responsibilities: own the model and the paged KV cache, turn a ``SchedulerOutput`` into
flat device inputs (one pinned staging buffer, one H2D copy per step), run the model
(eager for prefill / mixed batches, CUDA-graph replay for pure-decode batches at
bucketed batch sizes), sample, and read the sampled tokens back.

Every rank of a TP group runs the same runner on the same scheduler decisions (SPMD),
so no broadcast of inputs is needed; logits are all-gathered and sampling is
deterministic, which keeps ranks in lock step.

Parity: replaces upstream GPUModelRunner for the standalone engine (the reference patches
its batch reordering, vllm_metax/patch/performance/speculative_decode_perf.py:115-155, which
the scheduler here does natively).
"""
from __future__ import annotations

import time
from typing import Optional

import numpy as np
import torch

from .. import _custom_ops as ops
from .. import envs
from ..attention.metadata import AttentionMetadata, ForwardContext, set_forward_context
from ..config import EngineConfig
from ..layers.attention import PagedGQABackend
from ..parallel import state as ps
from .loader import build_model
from .scheduler import SchedulerOutput


def _graph_buckets(max_seqs: int) -> list[int]:
    b = [1, 2, 4, 8]
    b += list(range(16, 129, 16))
    b += list(range(160, 513, 32))
    return [x for x in b if x <= max_seqs] + ([max_seqs] if max_seqs not in b else [])


class ModelRunner:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        par = cfg.parallel
        ps.init_distributed(par.tensor_parallel_size, par.pipeline_parallel_size, par.data_parallel_size,
                            par.decode_context_parallel_size, device=cfg.device,
                            prefill_context_parallel_size=par.prefill_context_parallel_size)
        if cfg.device == "cuda":
            self.device = torch.device("cuda", ps.local_rank() if torch.cuda.device_count() > 1 else 0)
            torch.cuda.set_device(self.device)
            if not ops.load_native():
                raise RuntimeError("native library missing on a GPU box; run python -m vllm_metax_b200._build")
        else:
            self.device = torch.device("cpu")
        self.is_cuda = self.device.type == "cuda"
        torch.manual_seed(cfg.model.seed)
        ps.set_eplb(par.enable_eplb, par.num_redundant_experts)
        ps.set_moe_parallel(par.use_sequence_parallel_moe, par.all2all_backend)
        with torch.no_grad():
            self.model = build_model(cfg, self.device)
        self.eplb = None
        if par.enable_eplb:
            from ..layers.fused_moe import FusedMoE
            from ..parallel.eplb import EplbState

            moe = [m for m in self.model.modules() if isinstance(m, FusedMoE) and m.eplb]
            self.eplb = EplbState(moe, par.eplb_step_interval, par.eplb_window, par.eplb_log_balancedness)
        self.lora = None
        if cfg.model.enable_lora:
            from ..lora import LoRAManager

            self.lora = LoRAManager(self.model, cfg.model.max_loras, cfg.model.max_lora_rank, self.device, cfg.model.dtype)
        self.block_size = cfg.cache.block_size
        sc = cfg.scheduler
        self.max_tokens = max(sc.max_num_batched_tokens, sc.max_num_seqs)
        ps.set_max_tokens_per_step(self.max_tokens)
        self.max_seqs = sc.max_num_seqs
        # decode context parallel: a scheduler block of block_size * dcp tokens is block_size slots on every rank of the
        # DCP group (token p lives on rank p % dcp, at local index p // dcp)
        self.dcp = ps.get_dcp_group().world_size
        self.dcp_rank = ps.get_dcp_group().rank_in_group
        self.virt_bs = self.block_size * self.dcp
        if self.dcp > 1:
            m = cfg.model
            # GQA: the KV heads of a DCP group must be replicas of one another.  MLA: the latent cache is the same on
            # every tensor-parallel rank, so any dcp that divides tp works.
            reps = ps.tp_size() // m.num_key_value_heads if m.num_key_value_heads < ps.tp_size() else 1
            if not m.is_mla and reps % self.dcp != 0:
                raise ValueError("decode context parallelism needs a GQA model whose KV heads are replicated over at "
                                 f"least dcp tensor-parallel ranks (kv heads {m.num_key_value_heads}, tp {ps.tp_size()}, "
                                 f"dcp {self.dcp}), or an MLA model")
        self.dcp_per_token = self.dcp > 1 and cfg.model.is_mla
        self.cascade = bool(envs.B200_CASCADE_ATTENTION) and cfg.cache.enable_prefix_caching and self.dcp == 1
        self.uses_mrope = bool(getattr(self.model, "uses_mrope", False))
        # prefill context parallel: full model copies that split the tokens of every prefill chunk (parallel/pcp.py)
        self.pcp = ps.get_pcp_group().world_size
        if self.pcp > 1 and (self.dcp > 1 or getattr(cfg.model, "compress_ratios", None) is not None):
            raise ValueError("prefill context parallelism serves GQA and MLA models with an unsplit cache "
                             "(not combined with decode context parallelism or the DeepSeek-V4 compressed caches)")
        # pipeline parallel with overlapped steps: asynchronous stage-to-stage transfers and one token buffer per
        # step in flight
        import collections

        self._pp_async = ps.get_pp_group().world_size > 1 and envs.B200_PP_OVERLAP
        self._pp_sends: collections.deque = collections.deque()
        self._pp_next = 0
        self._prep_done = None
        self._pp_copy_stream = None
        self._pp_host = None
        self.max_blocks_per_seq = (sc.max_model_len + self.virt_bs - 1) // self.virt_bs
        self.kv_caches: list = []
        self.num_blocks = 0
        self._alloc_inputs()
        self._alloc_state_slots()
        self._enable_fused_tp()
        self.graphs: dict[int, tuple] = {}
        self.use_graphs = self.is_cuda and not cfg.enforce_eager and envs.B200_CUDA_GRAPHS
        # replicas that share their experts exchange tokens in every MoE layer with sizes agreed on the host, and
        # their steps differ in shape (one decodes while another prefills): a replayed graph would skip the host
        # handshake its peer is waiting in, so these engines run eagerly
        if ps.get_dp_group().world_size > 1 and cfg.model.is_moe:
            self.use_graphs = False
        self.launch_count = 0
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.is_cuda else 1

    def _enable_fused_tp(self) -> None:
        """Swap the row-parallel linears + all-reduce + add-norm of a TP model for the fused NVLink kernel."""
        inner = getattr(self.model, "model", None)
        self.fused_tp = False
        self.custom_ar = None
        if ps.tp_size() > 1 and self.is_cuda and envs.B200_CUSTOM_ALLREDUCE:
            from ..parallel.custom_allreduce import CustomAllReduce

            # small reductions (decode steps, MoE outputs, logits pieces) skip NCCL's launch + protocol latency
            self.custom_ar = CustomAllReduce(ps.get_tp_group(), self.device, envs.B200_CUSTOM_ALLREDUCE_MAX_BYTES)
            ok, why = self.custom_ar.self_test()    # checked once against an fp32 sum at this world size
            if ok:
                self.custom_ar.attach()
            else:
                import warnings

                warnings.warn(f"peer-store all-reduce failed its start-up check ({why}); "
                              "tensor-parallel reductions stay on NCCL")
                self.custom_ar = None
        if (ps.tp_size() == 1 or ps.get_pp_group().world_size > 1 or not envs.B200_FUSED_TP_COLLECTIVES
                or inner is None or not hasattr(inner, "forward_fused_tp")
                or not getattr(inner, "supports_fused_tp", True) or self.cfg.model.quantization
                or self.cfg.model.enable_lora):
            return
        from ..parallel.fused_collectives import get_fused_row_parallel

        fused = get_fused_row_parallel(ps.get_tp_group(), self.device, self.max_tokens,
                                       self.cfg.model.hidden_size, self.cfg.model.dtype)
        ok, why = fused.self_test()                 # same verdict on every rank
        if not ok and fused.nvls is not None:
            import warnings

            warnings.warn(f"fused row-parallel path failed its start-up check with the in-switch reduction ({why}); "
                          "retrying with the peer-store kernels at every step size")
            fused.disable_nvls()
            ok, why = fused.self_test()
        if not ok and fused.out_mc:
            import warnings

            warnings.warn(f"fused row-parallel path failed its start-up check with the multicast gather ({why}); "
                          "retrying with per-rank peer stores")
            fused.disable_multicast()
            ok, why = fused.self_test()
        if not ok:
            import warnings

            warnings.warn(f"fused row-parallel path failed its start-up check ({why}); "
                          "row-parallel layers use GEMM + all-reduce + add-norm")
            return
        inner.fused_ar = fused
        # the split path serves every step size; the single-kernel path only pays off on large steps
        inner.fused_min_tokens = envs.B200_FUSED_TP_MIN_TOKENS if fused.kernel == "mono" else 0
        self.fused_tp = True

    # ------------------------------------------------------------------ buffers
    def _alloc_inputs(self) -> None:
        dev, T, B, MB = self.device, self.max_tokens, self.max_seqs, self.max_blocks_per_seq
        # one int64 staging area: [input_ids T | positions T | slot_mapping T] and one int32 area
        self.n64 = 3 * T
        self.n32 = (B + 1) + B + B * MB + (B + 1)
        pin = self.is_cuda
        self.h64 = torch.zeros(self.n64, dtype=torch.int64, pin_memory=pin)
        self.h32 = torch.zeros(self.n32, dtype=torch.int32, pin_memory=pin)
        self.d64 = torch.zeros(self.n64, dtype=torch.int64, device=dev)
        self.d32 = torch.zeros(self.n32, dtype=torch.int32, device=dev)
        self.h64_np, self.h32_np = self.h64.numpy(), self.h32.numpy()
        self._bt_owner: list = [None] * B
        self.mrope_dev = torch.zeros(3, T, dtype=torch.int64, device=dev) if self.uses_mrope else None
        self.input_ids = self.d64[:T]
        self.positions = self.d64[T:2 * T]
        self.slot_mapping = self.d64[2 * T:3 * T]
        o = 0
        self.query_start_loc = self.d32[o:o + B + 1]; o += B + 1
        self.seq_lens = self.d32[o:o + B]; o += B
        self.block_table = self.d32[o:o + B * MB].view(B, MB); o += B * MB
        self.prefill_qsl = self.d32[o:o + B + 1]
        S = max(B, T)        # with draft tokens every fed position of a request is sampled
        self.sampled = torch.zeros(S, dtype=torch.int64, device=dev)
        self._pp_slots = [torch.zeros(S, dtype=torch.int64, device=dev)
                          for _ in range(2 * ps.get_pp_group().world_size)] if self._pp_async else []
        self.sampled_host = torch.zeros(S, dtype=torch.int64, pin_memory=pin)
        self.sample_idx = torch.zeros(S, dtype=torch.int64, device=dev)
        self.sample_idx_host = torch.zeros(S, dtype=torch.int64, pin_memory=pin)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def kv_bytes_per_block(self) -> int:
        spec = self.model.kv_cache_spec()
        n = self.model.num_kv_layers()
        from ..layers.attention import KV_DTYPES

        if spec["kind"] == "gqa":
            from ..ops import turboquant as tq

            if tq.is_turboquant(self.cfg.cache.kv_cache_dtype):
                slot = tq.TqFormat.from_name(self.cfg.cache.kv_cache_dtype).slot_bytes
                return self.block_size * spec["num_kv_heads"] * slot * n
            dt = KV_DTYPES[self.cfg.cache.kv_cache_dtype] or self.cfg.model.dtype
            per = 2 * self.block_size * spec["num_kv_heads"] * spec["head_size"] * torch.empty((), dtype=dt).element_size()
            if self.cfg.cache.kv_cache_dtype.endswith("per_token_head"):
                per += 2 * self.block_size * spec["num_kv_heads"] * 4
            return per * n
        return self.model.kv_bytes_per_block(self.block_size, self.cfg.cache.kv_cache_dtype)

    def determine_num_blocks(self) -> int:
        c = self.cfg.cache
        if c.num_gpu_blocks:
            return c.num_gpu_blocks
        if not self.is_cuda:
            return 512
        torch.cuda.synchronize()
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - int(total * (1.0 - c.gpu_memory_utilization)) - (6 << 30)  # activation head-room
        n = max(16, budget // max(1, self.kv_bytes_per_block()))          # attention-free models: blocks only meter length
        want = self.max_seqs * self.max_blocks_per_seq
        return int(min(n, max(want, 64)))

    def init_kv_cache(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        spec = self.model.kv_cache_spec()
        if spec["kind"] == "gqa":
            self.kv_caches = [
                PagedGQABackend.allocate(num_blocks, self.block_size, spec["num_kv_heads"], spec["head_size"],
                                         self.cfg.model.dtype, self.cfg.cache.kv_cache_dtype, self.device)
                for _ in range(self.model.num_kv_layers())]
        else:
            self.kv_caches = self.model.allocate_kv_cache(num_blocks, self.block_size, self.cfg.cache.kv_cache_dtype,
                                                          self.device)

    # ------------------------------------------------------------------ per-request recurrent state (hybrid models)
    def _alloc_state_slots(self) -> None:
        """Models with recurrent layers (gated delta rule, short convolutions) keep one state slot per running request
        next to the paged KV cache.  Slot ``max_seqs`` is scratch: CUDA-graph padding rows read and write it."""
        self.state_slots: Optional[dict] = None
        if not hasattr(self.model, "allocate_state"):
            return
        B = self.max_seqs
        self.state_bytes = self.model.allocate_state(B + 1, self.device)
        self.state_slots = {}
        self.free_state_slots = list(range(B - 1, -1, -1))
        pin = self.is_cuda
        self.state_host = torch.zeros(2 * B, dtype=torch.int32, pin_memory=pin)
        self.state_dev = torch.zeros(2 * B, dtype=torch.int32, device=self.device)
        self.state_dev[:B].fill_(B)

    def release_request(self, req) -> None:
        """Called when a request gives its KV blocks back (finished, aborted or preempted for re-computation)."""
        if self.state_slots is not None:
            slot = self.state_slots.pop(req.request_id, None)
            if slot is not None:
                self.free_state_slots.append(slot)

    def _state_metadata(self, so: SchedulerOutput, md: AttentionMetadata, B_eff: int) -> None:
        B = self.max_seqs
        h = self.state_host.numpy()
        for i, s in enumerate(so.scheduled):
            rid = s.request.request_id
            slot = self.state_slots.get(rid)
            if slot is None:
                slot = self.state_slots[rid] = self.free_state_slots.pop()
            h[i] = slot
            h[B + i] = 1 if s.start_pos > 0 else 0
        n = len(so.scheduled)
        h[n:B_eff] = B
        h[B + n: B + B_eff] = 0
        self.state_dev[:B_eff].copy_(self.state_host[:B_eff], non_blocking=True)
        self.state_dev[B: B + B_eff].copy_(self.state_host[B: B + B_eff], non_blocking=True)
        md.extra["state_indices"] = self.state_dev[:B_eff]
        md.extra["state_has_init"] = self.state_dev[B: B + B_eff]

    # ------------------------------------------------------------------ multimodal inputs
    @torch.no_grad()
    def encode_multimodal(self, prompt_token_ids: list, mm: dict):
        """Run the model's encoder on a request's images and line the features up with the prompt's placeholder tokens.

        ``mm["image"]``: one image or a list of them (PIL, ``[3, H, W]`` tensors) or pre-processed ``pixel_values
        [n, 3, S, S]``.  The prompt holds either one placeholder token per image (expanded here to the encoder's token
        count) or the already expanded run.  Returns ``(token ids, (features [N, hidden], positions [N], hash))``."""
        import hashlib

        model = self.model
        if not getattr(model, "is_multimodal", False):
            raise ValueError(f"{self.cfg.model.architecture} takes no multi-modal inputs")
        if hasattr(model, "encode_request"):         # models with their own input layout (dynamic-resolution towers)
            ids, triple, extras = model.encode_request(list(prompt_token_ids), mm, self.device)
            return ids, (*triple, extras)
        imgs = mm.get("pixel_values", mm.get("image"))
        if isinstance(imgs, torch.Tensor) and imgs.dim() == 4:
            pixels = imgs
        else:
            if not isinstance(imgs, (list, tuple)):
                imgs = [imgs]
            pixels = torch.stack([model.preprocess(im) for im in imgs])
        feats = model.embed_multimodal(pixels.to(self.device))              # [n, per, hidden]
        n, per, hid = feats.shape
        tok = model.image_token_id
        count = sum(1 for t in prompt_token_ids if t == tok)
        if count == n and per > 1:
            ids = []
            for t in prompt_token_ids:
                ids.extend([tok] * per if t == tok else [t])
        elif count == n * per:
            ids = prompt_token_ids
        else:
            raise ValueError(f"prompt has {count} image placeholder tokens for {n} image(s) of {per} tokens each")
        pos = np.asarray([i for i, t in enumerate(ids) if t == tok], dtype=np.int64)
        digest = hashlib.sha256(pixels.detach().float().cpu().numpy().tobytes()).hexdigest()[:16]
        return ids, (feats.reshape(n * per, hid), pos, digest)

    def _multimodal_rows(self, so: SchedulerOutput, md: AttentionMetadata) -> None:
        """Rows of this step's flat batch that are placeholder tokens, with their features in the same order."""
        rows, parts, t = [], [], 0
        for s in so.scheduled:
            r = s.request
            if r.mm_embeds is not None and s.start_pos < r.mm_positions[-1] + 1:
                lo = int(np.searchsorted(r.mm_positions, s.start_pos))
                hi = int(np.searchsorted(r.mm_positions, s.start_pos + s.num_new_tokens))
                if hi > lo:
                    rows.append(r.mm_positions[lo:hi] - s.start_pos + t)
                    parts.append(r.mm_embeds[lo:hi])
            t += s.num_new_tokens
        if rows:
            md.extra["mm_rows"] = torch.from_numpy(np.concatenate(rows)).to(self.device)
            md.extra["mm_embeds"] = torch.cat(parts) if len(parts) > 1 else parts[0]

    # ------------------------------------------------------------------ input prep
    def _prepare(self, so: SchedulerOutput, pad_to: int = 0, copy: bool = True):
        """Fills the pinned staging areas for ``so`` and (``copy``) sends them to the device.  With ``copy=False`` the
        transfer is left to ``_submit_inputs`` - the step is being prepared while the device still runs the previous
        one, and token ids that are not known yet are written by ``_refill_tokens`` first."""
        T_, B_, MB = self.max_tokens, self.max_seqs, self.max_blocks_per_seq
        ids, pos, slots = self.h64_np[:T_], self.h64_np[T_:2 * T_], self.h64_np[2 * T_:3 * T_]
        o = 0
        qsl = self.h32_np[o:o + B_ + 1]; o += B_ + 1
        sl = self.h32_np[o:o + B_]; o += B_
        bt = self.h32_np[o:o + B_ * MB].reshape(B_, MB); o += B_ * MB
        pqsl = self.h32_np[o:o + B_ + 1]
        bs = self.block_size
        d, dr, vbs = self.dcp, self.dcp_rank, self.virt_bs
        owners = self._bt_owner          # per staging row: (request, blocks already written), None = unknown
        ctx_local = []
        vis_local, tok_req = [], []
        t = 0
        qsl[0] = 0
        max_q = max_seq = 0
        sample_rows = []
        sample_reqs = []
        # decode rows first (the scheduler's order): one token each, filled as whole arrays
        nd_fast = 0
        if d == 1 and so.num_decode and so.scheduled[so.num_decode - 1].num_new_tokens == 1 and all(
                s.num_spec == 0 for s in so.scheduled[: so.num_decode]):
            nd_fast = so.num_decode
            dec = so.scheduled[:nd_fast]
            p0s = [s.start_pos for s in dec]
            ids[:nd_fast] = [s.request.token_at(p) for s, p in zip(dec, p0s)]
            pos[:nd_fast] = p0s
            slots[:nd_fast] = [s.request.block_ids[p // bs] * bs + p % bs for s, p in zip(dec, p0s)]
            qsl[1:nd_fast + 1] = np.arange(1, nd_fast + 1, dtype=np.int32)
            sl[:nd_fast] = np.asarray(p0s, dtype=np.int32) + 1
            max_q, max_seq = 1, max(p0s) + 1
            for i, s in enumerate(dec):
                r = s.request
                nb = len(r.block_ids)
                own = owners[i]
                if own is not None and own[0] is r and own[1] <= nb:
                    if own[1] < nb:
                        bt[i, own[1]:nb] = r.block_ids[own[1]:]
                        owners[i] = (r, nb)
                else:
                    bt[i, :nb] = r.block_ids
                    owners[i] = (r, nb)
                if s.samples:
                    sample_rows.append(i)
                    sample_reqs.append(r)
            t = nd_fast
        for i, s in enumerate(so.scheduled):
            if i < nd_fast:
                continue
            r = s.request
            n, p0 = s.num_new_tokens, s.start_pos
            if d > 1:
                ids[t:t + n] = ((r.all_token_ids + r.spec_token_ids[: s.num_spec])[p0:p0 + n] if s.num_spec
                                else r.all_token_ids[p0:p0 + n])
                ar = np.arange(p0, p0 + n)
                pos[t:t + n] = ar
                blk = np.asarray(r.block_ids, dtype=np.int64)
                slots[t:t + n] = np.where(ar % d == dr, blk[ar // vbs] * bs + (ar % vbs) // d, -1)
                ctx_local.append(max(0, (p0 - dr + d - 1) // d))
                if self.dcp_per_token:      # MLA: cache entries of this rank that token p may see, (p - dr + d) // d
                    vis_local.append((ar - dr + d) // d)
                    tok_req.append(np.full(n, i, dtype=np.int64))
            elif n == 1:
                ids[t] = r.token_at(p0)
                pos[t] = p0
                slots[t] = r.block_ids[p0 // bs] * bs + p0 % bs
            else:
                if s.num_spec:
                    toks = (r.all_token_ids + r.spec_token_ids[: s.num_spec])[p0:p0 + n]
                else:
                    toks = r.all_token_ids[p0:p0 + n] if r.output_token_ids else r.prompt_token_ids[p0:p0 + n]
                ids[t:t + n] = toks
                ar = np.arange(p0, p0 + n)
                pos[t:t + n] = ar
                blk = np.asarray(r.block_ids, dtype=np.int64)
                slots[t:t + n] = blk[ar // bs] * bs + ar % bs
            t += n
            qsl[i + 1] = t
            sl[i] = p0 + n if d == 1 else max(0, (p0 + n - dr + d - 1) // d)     # tokens in THIS rank's cache
            nb = len(r.block_ids)
            own = owners[i]
            if own is not None and own[0] is r and own[1] <= nb:      # same request in this row: only its new blocks
                if own[1] < nb:
                    bt[i, own[1]:nb] = r.block_ids[own[1]:]
                    owners[i] = (r, nb)
            else:
                bt[i, :nb] = r.block_ids
                owners[i] = (r, nb)
            max_q = max(max_q, n)
            max_seq = max(max_seq, p0 + n)
            if s.samples:
                for row in range(t - 1 - s.num_spec, t):      # drafts: every fed position is verified
                    sample_rows.append(row)
                    sample_reqs.append(r)
        B = len(so.scheduled)
        nd = so.num_decode
        if pad_to > B:  # graph padding: dummy decodes that write nowhere and read block 0
            for i in range(B, pad_to):
                ids[t] = 0; pos[t] = 0; slots[t] = -1
                t += 1
                qsl[i + 1] = t
                sl[i] = 1
                bt[i, 0] = 0
                owners[i] = None
            B_eff, nd_eff = pad_to, pad_to
        else:
            B_eff, nd_eff = B, nd
        pqsl[: B_eff - nd_eff + 1] = qsl[nd_eff:B_eff + 1] - qsl[nd_eff]
        T = t
        self._staged = (T, B_eff)
        if copy:
            self._submit_inputs()
        md = AttentionMetadata(
            num_tokens=T, num_reqs=B_eff, num_decodes=nd_eff, num_decode_tokens=nd_eff,
            query_start_loc=self.query_start_loc[:B_eff + 1], seq_lens=self.seq_lens[:B_eff],
            block_table=self.block_table[:B_eff], slot_mapping=self.slot_mapping[:T], max_query_len=max_q,
            max_seq_len=max_seq, block_size=bs, prefill_query_start_loc=self.prefill_qsl[:B_eff - nd_eff + 1],
            max_prefill_query_len=max_q if B_eff > nd_eff else 0)
        # MLA: prefill requests without cached context may take the up-projected MHA path
        md.extra["prefill_no_context"] = all(s.start_pos == 0 for s in so.scheduled[nd:])
        if self.cascade and B >= 2 and pad_to <= B:
            self._cascade_metadata(so, md, T)
        if d > 1:
            ctx_local += [0] * (B_eff - len(ctx_local))
            md.extra["dcp_ctx_lens"] = torch.tensor(ctx_local, dtype=torch.int32).to(self.device, non_blocking=True)
            md.extra["dcp_any_context"] = any(s.start_pos > 0 for s in so.scheduled[nd:])
            if self.dcp_per_token and vis_local and T > B_eff:      # steps with multi-token requests only
                vis = np.concatenate(vis_local + [np.ones(T - sum(len(v) for v in vis_local), dtype=np.int64)])
                req = np.concatenate(tok_req + [np.arange(B, B + T - sum(len(v) for v in tok_req), dtype=np.int64)])
                md.extra["dcp_vis_lens"] = torch.from_numpy(vis.astype(np.int32)).to(self.device, non_blocking=True)
                md.extra["dcp_token_req"] = torch.from_numpy(req).to(self.device, non_blocking=True)
        if self.state_slots is not None:
            self._state_metadata(so, md, B_eff)
        if getattr(self.model, "is_multimodal", False):
            self._multimodal_rows(so, md)
        if self.uses_mrope:
            self._mrope_positions(so, md, T)
        return md, T, sample_rows, sample_reqs

    def _mrope_positions(self, so: SchedulerOutput, md: AttentionMetadata, T: int) -> None:
        """The three rotary position streams of this step's tokens (``[3, T]``, a static buffer so that captured decode
        graphs read the current values): the request's prompt table where it has one, else position + offset."""
        out = np.empty((3, T), dtype=np.int64)
        t = 0
        for s in so.scheduled:
            r, n, p0 = s.request, s.num_new_tokens, s.start_pos
            ar = np.arange(p0, p0 + n)
            tab = r.mrope_positions
            if tab is None:
                out[:, t:t + n] = ar
            else:
                L = tab.shape[1]
                k = max(0, min(n, L - p0))
                if k:
                    out[:, t:t + k] = tab[:, p0:p0 + k]
                if k < n:
                    out[:, t + k:t + n] = ar[k:] + r.mrope_delta
            t += n
        if t < T:                      # graph padding rows
            out[:, t:] = 0
        self.mrope_dev[:, :T].copy_(torch.from_numpy(out), non_blocking=False)
        md.extra["mrope_positions"] = self.mrope_dev[:, :T]

    def _cascade_applies(self, so: SchedulerOutput) -> bool:
        if len(so.scheduled) < 2:
            return False
        first = so.scheduled[0].request.block_ids
        n = min(min(s.start_pos for s in so.scheduled) // self.block_size, len(first))
        if n * self.block_size * (len(so.scheduled) - 1) < envs.B200_CASCADE_MIN_SAVED_TOKENS:
            return False
        return all(s.request.block_ids[:n] == first[:n] for s in so.scheduled[1:])

    def _cascade_metadata(self, so: SchedulerOutput, md: AttentionMetadata, T: int) -> None:
        """Leading cache blocks that ALL requests of the step share (the same physical blocks, from the prefix cache)
        and that hold computed context: the attention layers read them once for the whole step."""
        first = so.scheduled[0].request.block_ids
        n = min(min(s.start_pos for s in so.scheduled) // self.block_size, len(first))
        for s in so.scheduled[1:]:
            ids = s.request.block_ids
            k = 0
            while k < n and ids[k] == first[k]:
                k += 1
            n = k
            if n == 0:
                return
        tokens = n * self.block_size
        if tokens * (len(so.scheduled) - 1) < envs.B200_CASCADE_MIN_SAVED_TOKENS:
            return
        md.extra["cascade_blocks"] = n
        md.extra["cascade_seq_len"] = torch.tensor([tokens], dtype=torch.int32).to(self.device, non_blocking=True)
        md.extra["cascade_qsl"] = torch.tensor([0, T], dtype=torch.int32).to(self.device, non_blocking=True)
        # from the host staging arrays: the device copies of this step may not have been submitted yet
        B_, MB, nb = self.max_seqs, self.max_blocks_per_seq, len(so.scheduled)
        sl = self.h32_np[B_ + 1: 2 * B_ + 1]
        bt = self.h32_np[2 * B_ + 1: 2 * B_ + 1 + B_ * MB].reshape(B_, MB)
        md.extra["cascade_suffix_lens"] = torch.from_numpy(sl[:nb] - tokens).to(self.device, non_blocking=True)
        md.extra["cascade_suffix_table"] = torch.from_numpy(np.ascontiguousarray(bt[:nb, n:])).to(self.device,
                                                                                                non_blocking=True)
        self.cascade_steps = getattr(self, "cascade_steps", 0) + 1

    def _submit_inputs(self) -> None:
        """One H2D per staging area (only the used prefix of each segment)."""
        T, B_eff = self._staged
        T_, B_, MB = self.max_tokens, self.max_seqs, self.max_blocks_per_seq
        if self.is_cuda:
            for seg in range(3):
                self.d64[seg * T_: seg * T_ + T].copy_(self.h64[seg * T_: seg * T_ + T], non_blocking=True)
            n32 = (B_ + 1) + B_ + B_eff * MB
            self.d32[:n32].copy_(self.h32[:n32], non_blocking=True)
            o2 = (B_ + 1) + B_ + B_ * MB
            self.d32[o2:o2 + B_eff + 1].copy_(self.h32[o2:o2 + B_eff + 1], non_blocking=True)
            self.h2d_bytes += 3 * T * 8 + (n32 + B_eff + 1) * 4
        else:
            self.d64.copy_(self.h64)
            self.d32.copy_(self.h32)

    def _refill_tokens(self, so: SchedulerOutput) -> None:
        """A step prepared ahead of time held provisional tokens: write the real ids of every row, and switch off the
        cache writes of rows whose request has finished in the meantime (their results are dropped)."""
        T_ = self.max_tokens
        ids, slots = self.h64_np[:T_], self.h64_np[2 * T_:3 * T_]
        t = 0
        for s in so.scheduled:
            r, n, p0 = s.request, s.num_new_tokens, s.start_pos
            if r.status.finished:
                s.zombie = True
                slots[t:t + n] = -1
                self.zombie_rows = getattr(self, "zombie_rows", 0) + 1
            elif n == 1:
                ids[t] = r.token_at(p0)
            else:
                ids[t:t + n] = r.all_token_ids[p0:p0 + n] if r.output_token_ids else r.prompt_token_ids[p0:p0 + n]
            t += n

    # ------------------------------------------------------------------ a step in two halves (overlapped host work)
    def prepare_step(self, so: SchedulerOutput) -> dict:
        """Host half of a step: batch shape, staging buffers, metadata.  Nothing is sent to the device."""
        B = len(so.scheduled)
        bucket = 0
        if self.use_graphs and so.num_decode == B and B > 0 and self.graphs:
            bucket = next((b for b in self.buckets if b >= B), 0)
        if self.is_cuda and self._prep_done is not None:
            self._prep_done.synchronize()          # the previous step's H2D copies have read the staging areas
        md, T, rows, reqs = self._prepare(so, pad_to=bucket, copy=False)
        return {"so": so, "md": md, "T": T, "rows": rows, "reqs": reqs, "bucket": bucket, "staged": self._staged}

    @torch.no_grad()
    def launch_step(self, prep: dict) -> "LaunchedStep":
        """Device half: inputs, forward (graph replay for decode buckets), sampling, and the start of the token
        read-back.  Returns without waiting for the device."""
        so, md, T, rows, reqs, bucket = (prep[k] for k in ("so", "md", "T", "rows", "reqs", "bucket"))
        self._refill_tokens(so)
        self._staged = prep["staged"]
        self._submit_inputs()
        if self.is_cuda:
            self._prep_done = torch.cuda.Event()
            self._prep_done.record()
        B, n = len(so.scheduled), len(rows)
        all_greedy = all(r.params.greedy and not r.params.needs_penalties and not r.params.constrained for r in reqs)
        logits = None
        if bucket:
            g, logits, _ = self.graphs[bucket]
            g.replay()
            logits = logits[:B]
            tokens_dev = self.sampled[:B] if all_greedy else self._sample(logits, reqs)
        else:
            h = self._forward(md, T)
            if n == 0:
                return LaunchedStep(self, reqs, 0, None, None)
            if n == T:
                hs = h
            else:
                self.sample_idx_host[:n] = torch.as_tensor(rows)
                self.sample_idx[:n].copy_(self.sample_idx_host[:n], non_blocking=True)
                hs = h.index_select(0, self.sample_idx[:n])
            logits = self.model.compute_logits(hs)
            tokens_dev = ops.argmax(logits, self.sampled[:n]) if all_greedy else self._sample(logits, reqs)
        self.sampled_host[:n].copy_(tokens_dev[:n], non_blocking=True)
        done = None
        if self.is_cuda:
            done = torch.cuda.Event()
            done.record()
        self.d2h_bytes += n * 8
        want_lp = any(r.params.logprobs is not None for r in reqs)
        return LaunchedStep(self, reqs, n, done, logits if want_lp else None)

    # ------------------------------------------------------------------ execution
    def _forward(self, md: AttentionMetadata, T: int):
        ctx = ForwardContext(md, self.kv_caches, self.positions[:T])
        nvtx = self.is_cuda and envs.B200_NVTX
        if nvtx:      # a named range per step in Nsight timelines: tokens, decode / prefill split
            torch.cuda.nvtx.range_push(f"forward T={T} decodes={md.num_decodes} prefills={md.num_prefills}")
        try:
            with set_forward_context(ctx):
                pp = ps.get_pp_group()
                if pp.world_size == 1:
                    return self.model(self.input_ids[:T], self.positions[:T])
                inter = None if pp.is_first_rank else self._pp_recv(pp, T)
                out = self.model(self.input_ids[:T], self.positions[:T], inter)
                if isinstance(out, dict):
                    self._pp_send(pp, out)
                return out
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()

    # Pipeline stages exchange one tensor per step: [parts, T, hidden] with parts = hidden states (+ the residual
    # stream for pre-norm models).  Every stage runs the same scheduler, so shapes need no handshake.
    def _pp_parts(self) -> int:
        return 2 if getattr(self.model, "pp_residual", True) else 1

    def _pp_send(self, pp, out: dict) -> None:
        h, r = out["hidden_states"], out.get("residual")
        parts = [h] if self._pp_parts() == 1 else [h, r if r is not None else torch.zeros_like(h)]
        buf = torch.stack(parts).contiguous()
        if self._pp_async:      # the transfer runs beside the next step's forward; the buffer lives until it is done
            self._pp_sends.append((pp.isend(buf, pp.rank_in_group + 1), buf))
            while len(self._pp_sends) > 2 * pp.world_size:
                self._pp_sends.popleft()[0].wait()
        else:
            pp.send(buf, pp.rank_in_group + 1)

    def _pp_recv(self, pp, T: int) -> dict:
        buf = torch.empty(self._pp_parts(), T, self.cfg.model.hidden_size, dtype=self.cfg.model.dtype, device=self.device)
        if self._pp_async:
            pp.irecv(buf, pp.rank_in_group - 1).wait()
        else:
            pp.recv(buf, pp.rank_in_group - 1)
        return {"hidden_states": buf[0], "residual": buf[1] if buf.shape[0] > 1 else None}

    def _decode_splits(self, batch: int) -> int:
        spec = self.model.kv_cache_spec()
        if spec["kind"] != "gqa":
            return 1
        return ops.decode_num_splits(batch, spec["num_kv_heads"], self.cfg.scheduler.max_model_len, 1, self.sms)

    def _capture(self, bucket: int):
        """Capture a pure-decode step of `bucket` sequences: model -> logits -> arg-max."""
        md = AttentionMetadata(
            num_tokens=bucket, num_reqs=bucket, num_decodes=bucket, num_decode_tokens=bucket,
            query_start_loc=self.query_start_loc[:bucket + 1], seq_lens=self.seq_lens[:bucket],
            block_table=self.block_table[:bucket], slot_mapping=self.slot_mapping[:bucket], max_query_len=1,
            max_seq_len=self.cfg.scheduler.max_model_len, block_size=self.block_size,
            prefill_query_start_loc=self.prefill_qsl[:1], max_prefill_query_len=0)
        md.decode_num_splits = self._decode_splits(bucket)
        if self.dcp > 1:                      # decode rows of the captured step take the context-parallel path
            md.extra["dcp_ctx_lens"] = torch.zeros(bucket, dtype=torch.int32, device=self.device)
            md.extra["dcp_any_context"] = False
        if self.uses_mrope:
            md.extra["mrope_positions"] = self.mrope_dev[:, :bucket]
        if self.state_slots is not None:      # warm-up and capture run on the scratch slot
            B = self.max_seqs
            self.state_dev[:bucket].fill_(B)
            self.state_dev[B: B + bucket].zero_()
            md.extra["state_indices"] = self.state_dev[:bucket]
            md.extra["state_has_init"] = self.state_dev[B: B + bucket]
        spec = self.model.kv_cache_spec()
        if md.decode_num_splits > 1 and spec["kind"] == "gqa":
            hq = spec["num_kv_heads"] * (self.cfg.model.num_attention_heads // self.cfg.model.num_key_value_heads)
            md.decode_workspace = torch.empty(md.decode_num_splits * bucket * hq * (spec["head_size"] + 1),
                                              dtype=torch.float32, device=self.device)
        # safe dummy inputs for warm-up
        self.seq_lens[:bucket].fill_(1)
        self.slot_mapping[:bucket].fill_(-1)
        self.block_table[:bucket].zero_()
        self.positions[:bucket].zero_()
        self.input_ids[:bucket].zero_()
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                h = self._forward(md, bucket)
                logits = self.model.compute_logits(h)
                ops.argmax(logits, self.sampled[:bucket])
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if getattr(self, "_graph_pool", None) is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g, pool=self._graph_pool, stream=stream):
            h = self._forward(md, bucket)
            logits = self.model.compute_logits(h)
            ops.argmax(logits, self.sampled[:bucket])
        self.graphs[bucket] = (g, logits, md)

    def capture_graphs(self, buckets: Optional[list[int]] = None) -> None:
        if not self.use_graphs:
            return
        if ps.get_pp_group().world_size > 1:
            self.use_graphs = False
            return
        self.buckets = buckets or _graph_buckets(self.max_seqs)
        with torch.no_grad():
            for b in sorted(self.buckets, reverse=True):
                self._capture(b)
        ops.check_kernel_status(self.device.index or 0)

    @torch.no_grad()
    def _execute_pcp_sliced(self, so: SchedulerOutput) -> dict:
        """A step with prefill chunks under prefill context parallelism: this copy runs its slice of every chunk (and
        the small rows whole), the attention layers exchange K / V, the last copy samples and broadcasts."""
        from ..parallel import pcp as P

        g = ps.get_pcp_group()
        n_c, r = g.world_size, g.rank_in_group
        view = P.local_view(so, n_c, r)
        slots_all, sizes = P.gathered_slots(so, n_c, r, self.block_size)
        reqs_last = P.sampling_requests(so, n_c)
        self._route_lora(view)
        md, T, rows, reqs = self._prepare(view)
        md.extra["pcp_slots_all"] = torch.from_numpy(slots_all).to(self.device, non_blocking=True)
        md.extra["pcp_sizes"] = sizes
        h = self._forward(md, T)
        n = len(reqs_last)
        if n == 0:
            return {}
        if r == n_c - 1:
            assert [q.request_id for q in reqs] == [q.request_id for q in reqs_last]
            hs = h if n == T else h.index_select(0, torch.as_tensor(rows, dtype=torch.int64).to(self.device))
            logits = self.model.compute_logits(hs)
            greedy = all(q.params.greedy and not q.params.needs_penalties and not q.params.constrained for q in reqs)
            tokens = ops.argmax(logits, self.sampled[:n]) if greedy else self._sample(logits, reqs)
            if tokens.data_ptr() != self.sampled.data_ptr():
                self.sampled[:n].copy_(tokens[:n])
        g.broadcast(self.sampled[:n], src=n_c - 1)
        self.sampled_host[:n].copy_(self.sampled[:n], non_blocking=False)
        self.d2h_bytes += n * 8
        return {q.request_id: tok for q, tok in zip(reqs_last, self.sampled_host[:n].tolist())}

    @torch.no_grad()
    def execute(self, so: SchedulerOutput) -> dict[str, int]:
        if self.pcp > 1 and any(s.num_new_tokens >= self.pcp for s in so.scheduled):
            return self._execute_pcp_sliced(so)
        B = len(so.scheduled)
        pure_decode = so.num_decode == B and B > 0
        bucket = 0
        use_lora = self._route_lora(so)
        if self.use_graphs and pure_decode and self.graphs and not use_lora:      # adapter rows are gathered by index
            bucket = next((b for b in self.buckets if b >= B), 0)
            if bucket and self.cascade and self._cascade_applies(so):
                bucket = 0        # the shared prefix is worth more than the captured graph: this step runs eagerly
        md, T, rows, reqs = self._prepare(so, pad_to=bucket)
        all_greedy = all(r.params.greedy and not r.params.needs_penalties and not r.params.constrained for r in reqs)
        n = len(rows)
        logits = None
        if bucket:
            g, logits, _ = self.graphs[bucket]
            g.replay()
            logits = logits[:B]
            if all_greedy:
                tokens_dev = self.sampled[:B]
            else:
                tokens_dev = self._sample(logits, reqs)
        else:
            h = self._forward(md, T)
            if getattr(self, "keep_hidden", False):
                self.last_step = (h, md, T)      # draft proposers read the step's hidden states
            if n == 0:
                return {}
            pp = ps.get_pp_group()
            if isinstance(h, dict):  # non-last pipeline stage: the last stage samples and shares the tokens
                tokens_dev = pp.broadcast(self.sampled[:n], src=pp.world_size - 1)
            else:
                if n == T:
                    hs = h
                else:
                    self.sample_idx_host[:n] = torch.as_tensor(rows)
                    self.sample_idx[:n].copy_(self.sample_idx_host[:n], non_blocking=True)
                    hs = h.index_select(0, self.sample_idx[:n])
                logits = self.model.compute_logits(hs)
                tokens_dev = ops.argmax(logits, self.sampled[:n]) if all_greedy else self._sample(logits, reqs)
                if pp.world_size > 1:
                    if tokens_dev.data_ptr() != self.sampled.data_ptr():
                        self.sampled[:n].copy_(tokens_dev[:n])
                    tokens_dev = pp.broadcast(self.sampled[:n], src=pp.world_size - 1)
        if self.pcp > 1:        # the copies ran the same rows; the last copy's tokens are the step's
            if tokens_dev.data_ptr() != self.sampled.data_ptr():
                self.sampled[:n].copy_(tokens_dev[:n])
            tokens_dev = ps.get_pcp_group().broadcast(self.sampled[:n], src=self.pcp - 1)
        self.sampled_host[:n].copy_(tokens_dev[:n], non_blocking=False)
        self.d2h_bytes += n * 8
        toks = self.sampled_host[:n].tolist()
        if logits is not None and any(r.params.logprobs is not None for r in reqs):
            self._record_logprobs(logits, reqs, toks)
        out: dict = {}
        for r, tok in zip(reqs, toks):
            if r.request_id in out:                 # several verified positions of one request, in order
                prev = out[r.request_id]
                out[r.request_id] = (prev if isinstance(prev, list) else [prev]) + [tok]
            else:
                out[r.request_id] = tok
        for s in so.scheduled:                      # a drafted request always reports a list
            if s.num_spec and s.samples and not isinstance(out.get(s.request.request_id), list):
                out[s.request.request_id] = [out[s.request.request_id]]
        return out

    @torch.no_grad()
    def execute_dummy(self) -> None:
        """One forward pass over a single padding token that writes no KV and samples nothing: a replica without work
        still has to take part in the expert-parallel exchanges of the step the other replicas run."""
        self.input_ids[:1].zero_()
        self.positions[:1].zero_()
        self.slot_mapping[:1].fill_(-1)
        self.seq_lens[:1].fill_(1)
        self.query_start_loc[:2].copy_(torch.tensor([0, 1], dtype=torch.int32))
        self.block_table[:1].zero_()
        self.prefill_qsl[:1].zero_()
        md = AttentionMetadata(
            num_tokens=1, num_reqs=1, num_decodes=1, num_decode_tokens=1, query_start_loc=self.query_start_loc[:2],
            seq_lens=self.seq_lens[:1], block_table=self.block_table[:1], slot_mapping=self.slot_mapping[:1],
            max_query_len=1, max_seq_len=1, block_size=self.block_size, prefill_query_start_loc=self.prefill_qsl[:1],
            max_prefill_query_len=0)
        md.extra["prefill_no_context"] = True
        self._forward(md, 1)

    # ------------------------------------------------------------------ pipelined steps
    @torch.no_grad()
    def execute_async(self, so: SchedulerOutput) -> "PendingStep":
        """Launch one step without waiting for its tokens (pipeline parallel with one step per stage in flight).
        This stage's share of the step is enqueued - receive from the previous stage, forward, send to the next, or
        sample on the last stage - and the token broadcast from the last stage is started; ``PendingStep.result()``
        waits for it.  Steps launched back to back must hold disjoint requests (the scheduler's ``in_flight`` set).
        Upstream keeps ``pipeline_parallel_size`` batches in its executor queue the same way; the reference model
        files only mark the stage boundaries (vllm_metax/models/deepseek_v2.py:1364-1386, 1473-1494)."""
        pp = ps.get_pp_group()
        if self.is_cuda and self._prep_done is not None:
            self._prep_done.synchronize()          # the previous step's H2D copies have read the pinned staging area
        self._route_lora(so)
        md, T, rows, reqs = self._prepare(so)
        if self.is_cuda:
            self._prep_done = torch.cuda.Event()
            self._prep_done.record()
        all_greedy = all(r.params.greedy and not r.params.needs_penalties and not r.params.constrained for r in reqs)
        n = len(rows)
        h = self._forward(md, T)
        if n == 0:
            return PendingStep(self, None, None, [], 0)
        slot = self._pp_slots[self._pp_next % len(self._pp_slots)]
        self._pp_next += 1
        if not isinstance(h, dict):
            if n == T:
                hs = h
            else:
                idx = torch.as_tensor(rows, dtype=torch.int64)
                hs = h.index_select(0, idx.to(self.device, non_blocking=False))
            logits = self.model.compute_logits(hs)
            tokens = ops.argmax(logits, slot[:n]) if all_greedy else self._sample(logits, reqs)
            if tokens.data_ptr() != slot.data_ptr():
                slot[:n].copy_(tokens[:n])
        work = pp.broadcast_async(slot[:n], src=pp.world_size - 1) if pp.world_size > 1 else None
        return PendingStep(self, work, slot, reqs, n)

    def _route_lora(self, so: SchedulerOutput) -> bool:
        """Make the adapters of this step resident and tell the hooks which rows use which slot."""
        if self.lora is None:
            return False
        wanted = {s.request.lora_request.lora_int_id for s in so.scheduled if s.request.lora_request is not None}
        if not wanted:
            self.lora.set_batch(None)
            return False
        rows: list = []
        for s in so.scheduled:
            lr = s.request.lora_request
            slot = -1 if lr is None else self.lora.activate(lr, in_use=wanted)
            rows.extend([slot] * s.num_new_tokens)
        self.lora.set_batch(rows)
        return True

    def _record_logprobs(self, logits: torch.Tensor, reqs, toks: list) -> None:
        """Log-probability of every sampled token and of the ``logprobs`` most likely ones, appended to
        ``request.logprobs`` as ``{"token_id", "logprob", "top": [(token_id, logprob), ...]}`` (one entry per sampled
        position).  Taken from the raw logits: the distribution before temperature, top-k / top-p and penalties."""
        seen: dict = {}
        for r in reqs:
            seen[r.request_id] = seen.get(r.request_id, 0) + 1
        # a request with several sampled positions in one step is verifying drafts: not combined with logprobs
        rows = [i for i, r in enumerate(reqs) if r.params.logprobs is not None and seen[r.request_id] == 1
                and not r.status.finished]          # (a finished request's row was prepared ahead: nothing to record)
        if not rows:
            return
        idx = torch.as_tensor(rows, dtype=torch.int64, device=logits.device)
        lp = torch.log_softmax(logits.index_select(0, idx).float(), dim=-1)
        k = max(1, min(max(int(reqs[i].params.logprobs or 0) for i in rows), lp.shape[1]))
        top_v, top_i = lp.topk(k, dim=-1)
        chosen = lp.gather(1, torch.as_tensor([toks[i] for i in rows], dtype=torch.int64, device=logits.device)[:, None])
        top_v, top_i, chosen = top_v.cpu().tolist(), top_i.cpu().tolist(), chosen[:, 0].cpu().tolist()
        for j, i in enumerate(rows):
            n = int(reqs[i].params.logprobs or 0)
            reqs[i].logprobs.append({"token_id": int(toks[i]), "logprob": float(chosen[j]),
                                     "top": [(int(t), float(v)) for t, v in zip(top_i[j][:n], top_v[j][:n])]})

    def _sample(self, logits: torch.Tensor, reqs) -> torch.Tensor:
        from .sampler import sample_batch

        return sample_batch(logits, reqs, self.sampled[:len(reqs)])


class PendingStep:
    """Tokens of a launched step: ``result()`` waits for the last stage's broadcast and returns ``{request id: token}``
    (a list per request where several positions were sampled)."""

    def __init__(self, runner: ModelRunner, work, slot, reqs, n: int):
        self.runner, self.work, self.slot, self.reqs, self.n = runner, work, slot, reqs, n

    def result(self) -> dict:
        if self.n == 0:
            return {}
        if self.slot.is_cuda:
            # on a side stream: the host must not wait for the NEXT step's kernels, which are already queued on the
            # compute stream behind this step's
            r = self.runner
            if r._pp_copy_stream is None:
                r._pp_copy_stream = torch.cuda.Stream(device=r.device)
                r._pp_host = torch.zeros(self.slot.numel(), dtype=torch.int64, pin_memory=True)
            with torch.cuda.stream(r._pp_copy_stream):
                if self.work is not None:
                    self.work.wait()
                r._pp_host[: self.n].copy_(self.slot[: self.n], non_blocking=True)
            r._pp_copy_stream.synchronize()
            host = r._pp_host[: self.n]
        else:
            if self.work is not None:
                self.work.wait()
            host = self.slot[: self.n]
        self.runner.d2h_bytes += self.n * 8
        out: dict = {}
        for r, tok in zip(self.reqs, host.tolist()):
            if r.request_id in out:
                prev = out[r.request_id]
                out[r.request_id] = (prev if isinstance(prev, list) else [prev]) + [tok]
            else:
                out[r.request_id] = tok
        return out


class LaunchedStep:
    """A step whose device work has been queued; ``result()`` waits for its tokens: ``{request id: token}``."""

    def __init__(self, runner: ModelRunner, reqs, n: int, done, logits):
        self.runner, self.reqs, self.n, self.done, self.logits = runner, reqs, n, done, logits

    def result(self) -> dict:
        if self.n == 0:
            return {}
        if self.done is not None:
            self.done.synchronize()
        toks = self.runner.sampled_host[: self.n].tolist()
        if self.logits is not None:
            self.runner._record_logprobs(self.logits, self.reqs, toks)
        return {r.request_id: tok for r, tok in zip(self.reqs, toks)}
