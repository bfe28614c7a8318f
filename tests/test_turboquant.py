"""TurboQuant KV cache: the fp32 statement on CPU (error bounds of the format) and the CUDA kernels against it."""
import math
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from vllm_metax_b200.ops import turboquant as tq  # noqa: E402

gpu = pytest.mark.gpu
NAMES = list(tq.PRESETS)


def test_formats():
    f = tq.TqFormat.from_name("turboquant_4bit_nc")
    assert (f.kbits, f.vbits, f.nc, f.slot_bytes) == (4, 4, True, 144)
    assert tq.TqFormat.from_name("turboquant_3bit_nc").slot_bytes == 112
    assert tq.TqFormat.from_name("turboquant_k8v4").slot_bytes == 208
    assert tq.TqFormat.from_name("turboquant_4bit_nc").compression > 3.5
    assert tq.is_turboquant("turboquant_k3v4_nc") and not tq.is_turboquant("fp8") and not tq.is_turboquant(None)
    with pytest.raises(ValueError):
        tq.TqFormat.from_name("turboquant_2bit")
    h = tq.hadamard()
    torch.testing.assert_close(h @ h, torch.eye(128), rtol=0, atol=1e-5)
    torch.testing.assert_close(h, h.t())


@pytest.mark.parametrize("name", NAMES)
def test_reference_error_bounds(name):
    fmt = tq.TqFormat.from_name(name)
    g = torch.Generator().manual_seed(0)
    k = torch.randn(64, 2, 128, generator=g) * 3
    v = torch.randn(64, 2, 128, generator=g)
    kh, vh = tq.quant_dequant_ref(k, v, fmt)
    cos = torch.nn.functional.cosine_similarity(kh, k, dim=-1)
    assert cos.min() > {8: 0.995, 4: 0.98, 3: 0.95}[fmt.kbits]
    if fmt.nc:      # the reconstructed key keeps its length
        torch.testing.assert_close(kh.norm(dim=-1), k.norm(dim=-1), rtol=2e-3, atol=1e-3)
    step = (v.amax(-1) - v.amin(-1)) / ((1 << fmt.vbits) - 1)
    assert ((vh - v).abs().amax(-1) <= step * 0.51 + 2e-2).all()


def test_cpu_ops_round_trip():
    fmt = tq.TqFormat.from_name("turboquant_4bit_nc")
    g = torch.Generator().manual_seed(1)
    cache = tq.alloc_cache(4, 16, 2, fmt, "cpu")
    lens = [5, 33]
    bt = torch.tensor([[2, -1, -1], [1, 3, 0]], dtype=torch.int32)
    ks, vs = [], []
    for b, L in enumerate(lens):
        k = torch.randn(L, 2 * 128, generator=g)
        v = torch.randn(L, 2 * 128, generator=g)
        slots = tq._slots_of(bt[b], L, 16)
        tq.store(k, v, cache, slots, fmt)
        ks.append(k.reshape(L, 2, 128))
        vs.append(v.reshape(L, 2, 128))
    q = torch.randn(2, 8, 128, generator=g)
    got = tq.decode_attention(q, cache, bt, torch.tensor(lens), 0.09, fmt)
    exact = tq.decode_attention_ref(q, ks, vs, torch.tensor(lens), 0.09)
    assert torch.nn.functional.cosine_similarity(got.flatten(), exact.flatten(), dim=0) > 0.97


def _case(fmt, B=3, hkv=2, G=4, bs=16, lens=(1, 70, 333)):
    g = torch.Generator().manual_seed(2)
    nb = sum((L + bs - 1) // bs for L in lens) + 2
    perm = torch.randperm(nb, generator=g)
    mb = max((L + bs - 1) // bs for L in lens)
    bt = torch.zeros(B, mb, dtype=torch.int32)
    used = 0
    ks, vs, slots = [], [], []
    for b, L in enumerate(lens):
        n = (L + bs - 1) // bs
        bt[b, :n] = perm[used: used + n].int()
        used += n
        ks.append((torch.randn(L, hkv * 128, generator=g) * 2).to(torch.bfloat16))
        vs.append(torch.randn(L, hkv * 128, generator=g).to(torch.bfloat16))
        slots.append(tq._slots_of(bt[b], L, bs))
    q = torch.randn(B, hkv * G, 128, generator=g).to(torch.bfloat16)
    return nb, bs, hkv, bt, ks, vs, slots, q


@gpu
@pytest.mark.parametrize("name", NAMES)
def test_store_dequant_decode_kernels(name):
    fmt = tq.TqFormat.from_name(name)
    nb, bs, hkv, bt, ks, vs, slots, q = _case(fmt)
    cache = tq.alloc_cache(nb, bs, hkv, fmt, "cuda")
    assert cache.shape[-1] == torch.ops.b200.tq_slot_bytes(fmt.kbits, fmt.vbits)
    k_all, v_all, s_all = torch.cat(ks), torch.cat(vs), torch.cat(slots)
    s_in = s_all.clone()
    s_in[3] = -1                                     # a skipped token
    wide = torch.zeros(k_all.shape[0], k_all.shape[1] + 64, dtype=torch.bfloat16, device="cuda")
    wide[:, : k_all.shape[1]] = k_all.cuda()
    tq.store(wide[:, : k_all.shape[1]], v_all.cuda(), cache, s_in.cuda(), fmt)
    kd, vd = tq.dequant(cache, s_all.cuda(), fmt)
    k_ref, v_ref = tq.quant_dequant_ref(k_all.reshape(-1, hkv, 128), v_all.reshape(-1, hkv, 128), fmt)
    assert kd[3].abs().max() == 0 and vd[3].abs().max() == 0
    keep = torch.ones(s_all.numel(), dtype=torch.bool)
    keep[3] = False
    # a coordinate that sits on a level boundary may fall either way: compare vectors, not codes
    cos = torch.nn.functional.cosine_similarity(kd.float().cpu()[keep], k_ref[keep], dim=-1)
    assert cos.min() > 0.995, cos.min()
    # values: identical up to a code that sits exactly between two levels (one step apart, a handful of elements)
    dv = (vd.float().cpu()[keep] - v_ref[keep]).abs()
    step = ((v_ref[keep].amax(-1) - v_ref[keep].amin(-1)) / ((1 << fmt.vbits) - 1))[..., None]
    assert (dv <= step * 1.05 + 8e-2).all()
    assert (dv > 8e-2).float().mean() < 1e-3
    # decode: the kernel against attention over the kernel's own dequantised rows
    tq.store(k_all.cuda(), v_all.cuda(), cache, s_all.cuda(), fmt)
    kd, vd = tq.dequant(cache, s_all.cuda(), fmt, torch.bfloat16)
    lens = torch.tensor([k.shape[0] for k in ks])
    offs = [0] + lens.cumsum(0).tolist()
    kh = [kd[offs[b]: offs[b + 1]].float().cpu() for b in range(len(ks))]
    vh = [vd[offs[b]: offs[b + 1]].float().cpu() for b in range(len(ks))]
    want = tq.decode_attention_ref(q.float(), kh, vh, lens, 1 / math.sqrt(128))
    for splits in (1, 3):
        got = tq.decode_attention(q.cuda(), cache, bt.cuda(), lens.cuda(), 1 / math.sqrt(128), fmt, num_splits=splits)
        torch.testing.assert_close(got.float().cpu(), want, rtol=3e-2, atol=3e-2)
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", ["turboquant_k8v4", "turboquant_4bit_nc"])
def test_engine_runs_with_turboquant_cache(name):
    """The whole engine on CPU with a compressed cache: chunked prefill (context read back through the
    de-quantiser), decode from the slots, preemption-free run to the end."""
    from vllm_metax_b200 import LLM, ModelConfig, SamplingParams

    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=512, hidden_size=256, intermediate_size=512,
                      num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                      max_position_embeddings=256, dtype=torch.float32, seed=0)
    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks=32)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (40, 9)]       # 40 > 32: chunked prefill
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    base = LLM(cfg, **kw).generate(prompts, sp)
    llm = LLM(cfg, kv_cache_dtype=name, **kw)
    cache, fmt = llm.engine.runner.kv_caches[0]
    assert cache.dtype == torch.uint8 and cache.shape[-1] == fmt.slot_bytes
    outs = llm.generate(prompts, sp)
    assert [len(o.outputs[0].token_ids) for o in outs] == [6, 6]
    if name == "turboquant_k8v4":       # fp8 keys / 4-bit values barely move a greedy first token
        assert outs[0].outputs[0].token_ids[0] == base[0].outputs[0].token_ids[0]


@gpu
def test_engine_runs_with_turboquant_cache_gpu():
    from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
    from vllm_metax_b200 import _custom_ops as ops

    cfg = ModelConfig(architecture="LlamaForCausalLM", vocab_size=1024, hidden_size=512, intermediate_size=1024,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      max_position_embeddings=512, dtype=torch.bfloat16, seed=0)
    llm = LLM(cfg, device="cuda", kv_cache_dtype="turboquant_4bit_nc", block_size=16, max_model_len=256, max_num_seqs=4,
              max_num_batched_tokens=64, num_gpu_blocks=64)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (100, 9, 33)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [len(o.outputs[0].token_ids) for o in outs] == [12, 12, 12]
    torch.cuda.synchronize()
    ops.check_kernel_status(0)
