"""Tensor parallelism on CPU ranks (Gloo, world size 2): sharded weight loading from an HF-style
safetensors checkpoint, NCCL-style collectives path and the fused row-parallel path must both
reproduce the single-process greedy tokens."""
import json
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

HF_CFG = {"architectures": ["LlamaForCausalLM"], "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
          "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 512, "torch_dtype": "float32"}


def export_hf_checkpoint(model, path):
    """Write a single-process model as an HF-named safetensors checkpoint (q/k/v and gate/up unfused)."""
    from safetensors.torch import save_file

    cfg = model.cfg
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    out = {}
    for name, p in model.named_parameters():
        w = p.detach().clone()
        if "qkv_proj" in name:
            q, k, v = w.split([H * D, Hkv * D, Hkv * D], 0)
            for n, t in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                out[name.replace("qkv_proj", n)] = t.contiguous()
        elif "gate_up_proj" in name:
            if type(model.get_submodule(name.rsplit(".", 1)[0])).__name__ == "GateUpSiluLinear":   # rows interleaved
                g_, u_ = w[0::2], w[1::2]
            else:                                                                                   # [gate | up] halves
                g_, u_ = w[: w.shape[0] // 2], w[w.shape[0] // 2:]
            out[name.replace("gate_up_proj", "gate_proj")] = g_.contiguous()
            out[name.replace("gate_up_proj", "up_proj")] = u_.contiguous()
        elif name.endswith("embed_tokens.weight") or name.startswith("lm_head"):
            out[name] = w[: cfg.vocab_size].contiguous()
        else:
            out[name] = w.contiguous()
    os.makedirs(path, exist_ok=True)
    save_file(out, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(HF_CFG, f)


def _worker(rank, world, port, path, prompts, fused, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="1" if fused else "0",
                      B200_FUSED_TP_MIN_TOKENS="0")
    try:
        _worker_body(rank, world, path, prompts, fused, q)
    except BaseException as e:  # surface the failure to the parent instead of letting it time out
        if rank == 0:
            q.put(repr(e))
        raise


def _worker_body(rank, world, path, prompts, fused, q):
    from vllm_metax_b200 import LLM, SamplingParams

    llm = LLM(path, device="cpu", tensor_parallel_size=world, block_size=16, max_model_len=128, max_num_seqs=8,
              max_num_batched_tokens=64, num_gpu_blocks=64, dtype=torch.float32)
    assert llm.engine.runner.fused_tp == fused
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    if rank == 0:
        q.put([o.outputs[0].token_ids for o in outs])


@pytest.mark.parametrize("fused", [False, True])
def test_tp2_matches_single_process(tmp_path, fused):
    from vllm_metax_b200 import LLM, SamplingParams

    ref_llm = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=128, max_num_seqs=8,
                  max_num_batched_tokens=64, num_gpu_blocks=64)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (21, 40, 7)]
    want = [o.outputs[0].token_ids for o in ref_llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    path = str(tmp_path / "ckpt")
    export_hf_checkpoint(ref_llm.engine.runner.model, path)
    # the exported checkpoint round-trips through the loader
    again = LLM(path, device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64,
                num_gpu_blocks=64, dtype=torch.float32)
    assert [o.outputs[0].token_ids for o in again.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))] == want
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 200) + (50 if fused else 0)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, path, prompts, fused, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
