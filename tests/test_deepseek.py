"""DeepSeek V2/V3/V3.2: MLA (absorbed + MHA prefill), grouped routing, DSA indexer."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.ops import reference as ref

gpu = pytest.mark.gpu


def ds_cfg(**kw):
    d = dict(architecture="DeepseekV3ForCausalLM", vocab_size=512, hidden_size=256, intermediate_size=512,
             num_hidden_layers=3, num_attention_heads=4, q_lora_rank=96, kv_lora_rank=512, qk_nope_head_dim=32,
             qk_rope_head_dim=64, v_head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
             n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid", n_group=4, topk_group=2,
             topk_method="noaux_tc", routed_scaling_factor=2.5, norm_topk_prob=True, max_position_embeddings=256,
             dtype=torch.float32, seed=0)
    d.update(kw)
    return ModelConfig(**d)


KW = dict(block_size=16, max_model_len=128, max_num_seqs=4, num_gpu_blocks=64)


def test_mla_absorbed_equals_mha_prefill_cpu():
    """Chunked prefill (absorbed MQA over the cache) and one-shot prefill (up-projected MHA) agree."""
    a = LLM(ds_cfg(), device="cpu", max_num_batched_tokens=256, **KW)
    b = LLM(ds_cfg(), device="cpu", max_num_batched_tokens=16, **KW)
    b.engine.runner.model.load_state_dict(a.engine.runner.model.state_dict())
    b.engine.runner.model.finalize_weights()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (40, 23)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    assert [o.outputs[0].token_ids for o in a.generate(prompts, sp)] == [o.outputs[0].token_ids for o in b.generate(prompts, sp)]


def test_v32_indexer_full_topk_equals_dense_cpu():
    """With index_topk >= context length the sparse model must reproduce the dense one."""
    dense = LLM(ds_cfg(), device="cpu", max_num_batched_tokens=256, **KW)
    sparse = LLM(ds_cfg(architecture="DeepseekV32ForCausalLM", index_n_heads=16, index_head_dim=128, index_topk=64),
                 device="cpu", max_num_batched_tokens=256, **KW)
    sd = sparse.engine.runner.model.state_dict()
    sd.update(dense.engine.runner.model.state_dict())
    sparse.engine.runner.model.load_state_dict(sd)
    sparse.engine.runner.model.finalize_weights()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (30, 12)]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    assert [o.outputs[0].token_ids for o in dense.generate(prompts, sp)] == \
        [o.outputs[0].token_ids for o in sparse.generate(prompts, sp)]
    # and a small top-k still runs end to end
    small = LLM(ds_cfg(architecture="DeepseekV32ForCausalLM", index_n_heads=16, index_head_dim=128, index_topk=8),
                device="cpu", max_num_batched_tokens=256, **KW)
    out = small.generate(prompts, sp)
    assert all(len(o.outputs[0].token_ids) == 5 for o in out)


def test_ds_mla_record_roundtrip_cpu():
    kv_c, k_pe = torch.randn(7, 512), torch.randn(7, 64)
    rec = ref.pack_ds_mla(kv_c, k_pe)
    back = ref.unpack_ds_mla(rec)
    assert rec.shape == (7, 656)
    torch.testing.assert_close(back[:, 512:], k_pe.to(torch.bfloat16).float())
    assert (back[:, :512] - kv_c).abs().max() < 0.25


# ------------------------------------------------------------------ GPU
def _mla_case(lens, qlens, H, bs, fp8, seed=0):
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
    lat = torch.randn(total * bs, 576, generator=g)
    if fp8:
        cache = ref.pack_ds_mla(lat[:, :512], lat[:, 512:]).view(total, bs, 656)
    else:
        cache = lat.to(torch.bfloat16).view(total, bs, 576)
    T = sum(qlens)
    q = (torch.randn(T, H, 576, generator=g) * 0.3).to(torch.bfloat16)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    return q, cache, bt, torch.tensor(lens, dtype=torch.int32), qsl


@gpu
@pytest.mark.parametrize("H", [16, 128, 8, 32, 48])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("splits", [1, 3])
def test_mla_decode_gpu(H, fp8, splits, kernel_status_ok):
    q, cache, bt, sl, qsl = _mla_case([70, 300, 17, 1000], [1, 3, 1, 2], H, 64, fp8)
    lse = torch.empty(H, q.shape[0], device="cuda")
    got = ops.mla_decode(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), 0.1, query_start_loc=qsl.cuda(), lse_out=lse,
                         num_splits=splits)
    want, wlse = ref.mla_decode(q.float(), cache, bt, sl, 0.1, query_start_loc=qsl)
    a, b = got.float().cpu().flatten(), want.flatten()
    assert 1 - float(torch.dot(a, b) / (a.norm() * b.norm())) < 5e-4
    torch.testing.assert_close(lse.cpu(), wlse, rtol=2e-2, atol=2e-2)


@gpu
def test_mla_sparse_decode_gpu(kernel_status_ok):
    H, topk = 16, 64
    q, cache, bt, sl, qsl = _mla_case([200, 90, 500], [2, 1, 1], H, 64, True, seed=3)
    T = q.shape[0]
    g = torch.Generator().manual_seed(9)
    idx = torch.full((T, topk), -1, dtype=torch.int32)
    lims = [199, 200, 90, 500]
    for t in range(T):
        n = min(topk - 5, lims[t])
        idx[t, :n] = torch.randperm(lims[t], generator=g)[:n].to(torch.int32)
    got = ops.mla_decode(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), 0.1, query_start_loc=qsl.cuda(),
                         topk_indices=idx.cuda(), num_splits=1)
    want, _ = ref.mla_decode(q.float(), cache, bt, sl, 0.1, query_start_loc=qsl, topk_indices=idx)
    a, b = got.float().cpu().flatten(), want.flatten()
    assert 1 - float(torch.dot(a, b) / (a.norm() * b.norm())) < 5e-4


@gpu
@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("impl,bs,Hi,decode", [(1, 64, 64, False), (2, 64, 64, False), (2, 16, 32, False),
                                               (2, 128, 64, False), (2, 64, 64, True), (2, 32, 64, True)])
def test_indexer_logits_and_topk_gpu(int8, impl, bs, Hi, decode, kernel_status_ok):
    """impl 1: the mma.sync kernel, impl 2: the tcgen05 kernel (``kind::f8f6f4`` / ``kind::i8``); ``decode``: one query
    token per request, which the tcgen05 kernel serves with N = heads instead of 256."""
    lens, qlens = ([300, 1500, 64, 129], [1, 1, 1, 1]) if decode else ([300, 1500, 64], [5, 2, 64])
    g = torch.Generator().manual_seed(0)
    B = len(lens)
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + 1
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    perm = torch.randperm(total, generator=g)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o:o + nblk[b]].to(torch.int32)
        o += nblk[b]
    cache = torch.zeros(total, bs * 132, dtype=torch.uint8)
    for b in range(B):
        k = torch.randn(lens[b], 128, generator=g)
        pos = torch.arange(lens[b])
        slots = bt[b].long()[pos // bs] * bs + pos % bs
        ref.indexer_k_quant_and_cache(k, cache, slots, int8=int8)
        if b == 0:      # the CUDA writer produces the same bytes (a rounding tie may differ by one step)
            mine = torch.zeros_like(cache).cuda()
            ops.indexer_k_quant_and_cache(k.bfloat16().cuda(), mine, slots.cuda(), bs, False, int8)
            theirs = torch.zeros_like(cache)
            ref.indexer_k_quant_and_cache(k.bfloat16().float(), theirs, slots, int8=int8)
            assert (mine.cpu() != theirs).float().mean() < 2e-3
    T = sum(qlens)
    if int8:
        q = torch.randint(-127, 128, (T, Hi, 128), generator=g).to(torch.int8)
    else:
        q = (torch.randn(T, Hi, 128, generator=g)).to(torch.float8_e4m3fn)
    w = torch.randn(T, Hi, generator=g) * 0.1
    sl = torch.tensor(lens, dtype=torch.int32)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    topk = 128
    got, logits = ops.indexer_topk(q.cuda(), w.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), qsl.cuda(), topk, bs,
                                   max_seq_len=max(lens), return_logits=True, max_query_len=max(qlens), impl=impl)
    # oracle logits per token
    t = 0
    for b in range(B):
        kq, sc = ref.gather_indexer_k(cache, bt[b], lens[b], int8=int8)
        for i in range(qlens[b]):
            lim = lens[b] - qlens[b] + i + 1
            lg = ref.mqa_logits(q[t:t + 1].float(), kq, sc, w[t:t + 1], torch.tensor([0]), torch.tensor([lim]))[0]
            mine = logits[t, : lens[b]].cpu()
            fin = torch.isfinite(lg)
            assert bool((torch.isfinite(mine) == fin).all())
            tol = float(lg[fin].abs().max()) * 2e-3 + 2e-2          # int8 products are exact; sums reach 1e4
            torch.testing.assert_close(mine[fin], lg[fin], rtol=2e-2, atol=tol)
            # top-k: the selected set must be a valid top-k of the kernel's own logits
            sel = got[t].cpu()
            sel = sel[sel >= 0].long()
            kk = min(topk, lim)
            assert sel.numel() == kk and sel.unique().numel() == kk
            thr = torch.topk(mine[:lim], kk).values.min()
            assert bool((mine[sel] >= thr - 1e-6).all())
            t += 1


@gpu
def test_deepseek_v32_gpu_tracks_cpu(kernel_status_ok):
    from tests.test_e2e_gpu import lockstep

    cfg = dict(architecture="DeepseekV32ForCausalLM", hidden_size=512, num_attention_heads=16, qk_nope_head_dim=128,
               v_head_dim=128, q_lora_rank=256, moe_intermediate_size=256, intermediate_size=1024, index_n_heads=16,
               index_head_dim=128, index_topk=256, vocab_size=1024)
    kw = dict(block_size=64, max_model_len=512, max_num_seqs=4, max_num_batched_tokens=1024, num_gpu_blocks=32)
    cpu = LLM(ds_cfg(**cfg), device="cpu", **kw)
    gl = LLM(ds_cfg(**cfg, dtype=torch.bfloat16), device="cuda", enforce_eager=True, **kw)
    sd = {k: v.to(torch.bfloat16) if v.is_floating_point() and v.dtype != torch.float32 or v.dtype == torch.float32 and "bias" not in k else v
          for k, v in cpu.engine.runner.model.state_dict().items()}
    gl.engine.runner.model.load_state_dict({k: v for k, v in sd.items()})
    gl.engine.runner.model.finalize_weights()
    cpu.engine.runner.model.load_state_dict({k: v.float() for k, v in sd.items()})
    cpu.engine.runner.model.finalize_weights()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 60)]
    lockstep(cpu, gl, prompts, steps=4, tol=3e-2)


@gpu
def test_indexer_bf16_variant_gpu(kernel_status_ok):
    """Unquantised indexer: bf16 queries against a bf16 key cache, same logits / top-k contract."""
    bs, Hi = 64, 32
    lens, qlens = [200, 700], [3, 1]
    g = torch.Generator().manual_seed(3)
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + 1
    bt = torch.zeros(2, max(nblk), dtype=torch.int32)
    perm = torch.randperm(total, generator=g)
    bt[0, : nblk[0]] = perm[: nblk[0]].int()
    bt[1, : nblk[1]] = perm[nblk[0]: nblk[0] + nblk[1]].int()
    cache = torch.zeros(total, bs, 128, dtype=torch.bfloat16)
    for b in range(2):
        k = torch.randn(lens[b], 128, generator=g).bfloat16()
        pos = torch.arange(lens[b])
        cache.view(-1, 128)[bt[b].long()[pos // bs] * bs + pos % bs] = k
    T = sum(qlens)
    q = torch.randn(T, Hi, 128, generator=g).bfloat16()
    w = torch.randn(T, Hi, generator=g) * 0.1
    sl = torch.tensor(lens, dtype=torch.int32)
    qsl = torch.tensor([0, 3, 4], dtype=torch.int32)
    got, logits = ops.indexer_topk(q.cuda(), w.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), qsl.cuda(), 64, bs,
                                   max_seq_len=max(lens), return_logits=True)
    want = ref.sparse_attn_indexer(q.float(), w, cache, bt, sl, qsl, 64, bf16=True)
    t = 0
    for b in range(2):
        kq = cache[bt[b][: nblk[b]].long()].reshape(-1, 128)[: lens[b]].float()
        for i in range(qlens[b]):
            lim = lens[b] - qlens[b] + i + 1
            lg = ref.mqa_logits(q[t:t + 1].float(), kq, torch.ones(lens[b]), w[t:t + 1], torch.tensor([0]), torch.tensor([lim]))[0]
            mine = logits[t, : lens[b]].cpu()
            fin = torch.isfinite(lg)
            assert bool((torch.isfinite(mine) == fin).all())
            torch.testing.assert_close(mine[fin], lg[fin], rtol=2e-2, atol=5e-2)
            assert set(got[t].cpu().tolist()) - {-1} == set(want[t].tolist()) - {-1} or lim > 64
            t += 1


def test_deepseek_graph_under_another_architecture_name_cpu():
    """A checkpoint whose config names its own architecture but is the DeepSeek-V3 graph (MLA fields + a model type of
    that lineage) is served by the DeepSeek class."""
    d = dict(architectures=["JoyAILLMFlashForCausalLM"], model_type="joyai_llm_flash", vocab_size=512, hidden_size=128,
             intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, q_lora_rank=48, kv_lora_rank=512,
             qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32, n_routed_experts=8, num_experts_per_tok=2,
             moe_intermediate_size=64, n_shared_experts=1, n_group=2, topk_group=1, first_k_dense_replace=1,
             max_position_embeddings=256, torch_dtype="float32")
    mc = ModelConfig.from_hf_dict(d)
    assert mc.architecture == "DeepseekV3ForCausalLM" and mc.is_mla and mc.scoring_func == "sigmoid"
    out = LLM(mc, device="cpu", **KW).generate([[1, 2, 3, 4]], SamplingParams(max_tokens=3, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 3
    other = ModelConfig.from_hf_dict(dict(d, model_type="something_else", architectures=["LlamaForCausalLM"]))
    assert other.architecture == "LlamaForCausalLM"


def test_mla_tcgen05_tiling_arithmetic_cpu():
    """The index arithmetic of csrc/mla_decode_tcgen05.cu restated: for every visible length, split count and page
    size the kernel serves, the 32-token tiles of all splits cover the visible positions exactly once, no tile
    straddles a page, every tile holds at least one visible position, and TMA coordinates stay 16-byte aligned."""
    import random

    BN = 32
    rng = random.Random(0)
    for _ in range(2000):
        block_size = rng.choice([32, 64, 128, 256])
        max_blocks = rng.randint(1, 40)
        lim = min(rng.randint(-3, max_blocks * block_size + 40), max_blocks * block_size)      # the kernel clamps to the table
        splits = rng.randint(1, 9)
        tiles_total = (lim + BN - 1) // BN if lim > 0 else 0
        per = (tiles_total + splits - 1) // splits
        seen = []
        for s in range(splits):
            begin = s * per
            n = max(0, min(tiles_total, begin + per) - begin)
            for j in range(n):
                tok0 = (begin + j) * BN
                page_index, off = tok0 // block_size, tok0 % block_size
                assert page_index < max_blocks and off + BN <= block_size          # inside the table, inside one page
                assert tok0 < lim                                                  # at least one visible position
                seen.extend(range(tok0, min(tok0 + BN, lim)))
        assert seen == list(range(max(lim, 0)))
    # TMA: innermost coordinate c * 64 elements of 2 bytes = multiples of 128 bytes; boxes of 64 elements = 128 bytes
    assert all((c * 64 * 2) % 16 == 0 for c in range(9)) and (64 * 2) % 16 == 0 and (576 * 2) % 16 == 0
    # shared memory: Q tile + two cache stages + barriers fit the 227 KB limit with the 1024-byte alignment slack
    assert 128 * 576 * 2 + 2 * 32 * 576 * 2 + 10 * 8 + 16 + 1024 <= 232448
    # tensor memory: two score buffers of 32 fp32 columns and 256 output columns fit 512 columns
    assert 2 * 32 + 256 <= 512
