"""Multi-LoRA: requests with an adapter must generate exactly what a model with the adapter merged into its
weights generates; adapters share a batch with each other and with base-model requests."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402
from tests.test_tp_cpu import export_hf_checkpoint  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)
PROJ = {"self_attn": ["q_proj", "k_proj", "v_proj", "o_proj"], "mlp": ["gate_proj", "up_proj", "down_proj"]}


def make_adapter(base: dict, rank: int, seed: int, targets=None) -> dict:
    """Random adapter in PEFT naming for every targeted projection of the exported base checkpoint."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, w in base.items():
        parts = name.split(".")
        if len(parts) < 2 or not parts[-2].endswith("_proj"):
            continue
        if targets is not None and parts[-2] not in targets:
            continue
        stem = "base_model.model." + ".".join(parts[:-1])
        out[f"{stem}.lora_A.weight"] = torch.randn(rank, w.shape[1], generator=g) * 0.06
        out[f"{stem}.lora_B.weight"] = torch.randn(w.shape[0], rank, generator=g) * 0.06
    return out


def merged(base: dict, adapter: dict, alpha: float) -> dict:
    out = dict(base)
    for k, a in adapter.items():
        if ".lora_A." in k:
            b = adapter[k.replace("lora_A", "lora_B")]
            name = k[len("base_model.model."):].replace(".lora_A.weight", ".weight")
            out[name] = base[name] + (alpha / a.shape[0]) * (b @ a)
    return out


def test_lora_model_parsing():
    from vllm_metax_b200.lora import LoRAModel

    t = {"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": torch.zeros(8, 256),
         "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": torch.zeros(256, 8),
         "base_model.model.model.layers.0.mlp.down_proj.lora_A.default.weight": torch.zeros(8, 512),
         "base_model.model.model.layers.0.mlp.down_proj.lora_B.default.weight": torch.zeros(256, 8)}
    m = LoRAModel.from_tensors(t, {"lora_alpha": 16})
    assert m.rank == 8 and m.scaling == 2.0
    assert set(m.weights) == {("model.layers.0.self_attn", "qkv_proj"), ("model.layers.0.mlp", "down_proj")}
    assert set(m.weights[("model.layers.0.self_attn", "qkv_proj")]) == {"q"}
    with pytest.raises(ValueError):
        LoRAModel.from_tensors({"foo": torch.zeros(1)})


def test_lora_matches_merged_weights(tmp_path):
    from safetensors.torch import load_file, save_file

    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.lora import LoRARequest

    llm = LLM(tiny_cfg(), enable_lora=True, max_loras=2, max_lora_rank=8, enable_prefix_caching=True, **KW)
    assert llm.engine.runner.lora is not None
    d = str(tmp_path / "base")
    export_hf_checkpoint(llm.engine.runner.model, d)
    base = load_file(os.path.join(d, "model.safetensors"))
    ad1 = make_adapter(base, 8, 1)
    ad2 = make_adapter(base, 4, 2, targets={"q_proj", "v_proj", "down_proj"})
    ad3 = make_adapter(base, 8, 3, targets={"o_proj", "gate_proj"})
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 70, 9)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)

    def reference(adapter, alpha):
        dd = str(tmp_path / f"m{alpha}_{len(adapter)}")
        os.makedirs(dd)
        save_file(merged(base, adapter, alpha), os.path.join(dd, "model.safetensors"))
        import shutil

        shutil.copy(os.path.join(d, "config.json"), dd)
        return [o.outputs[0].token_ids for o in LLM(dd, dtype=torch.float32, **KW).generate(prompts, sp)]

    want0 = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    want1, want2, want3 = reference(ad1, 16), reference(ad2, 4), reference(ad3, 8)
    assert want1 != want0 and want2 != want0
    r1 = LoRARequest("a1", 1, tensors=ad1, config={"lora_alpha": 16})
    r2 = LoRARequest("a2", 2, tensors=ad2, config={"lora_alpha": 4})
    r3 = LoRARequest("a3", 3, tensors=ad3, config={"lora_alpha": 8})
    got1 = [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=r1)]
    assert got1 == want1
    # one batch: adapter 1, adapter 2 and the base model side by side (same prompt: the prefix cache must not mix them)
    mixed = llm.generate([prompts[1]] * 3, sp, lora_request=[r1, r2, None])
    assert [o.outputs[0].token_ids for o in mixed] == [want1[1], want2[1], want0[1]]
    # a third adapter evicts the least recently used slot; the evicted one reloads on demand
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=r3)] == want3
    assert len(llm.engine.runner.lora.list_adapters()) == 2
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp, lora_request=r1)] == want1
    with pytest.raises(ValueError):
        LLM(tiny_cfg(), **KW).generate(prompts[:1], sp, lora_request=r1)


def _tp_worker(rank, world, port, base_dir, adapter, prompts, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.lora import LoRARequest

    llm = LLM(base_dir, dtype=torch.float32, tensor_parallel_size=world, enable_lora=True, max_loras=2, max_lora_rank=8, **KW)
    assert not llm.engine.runner.fused_tp
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True),
                        lora_request=LoRARequest("a", 1, tensors=adapter, config={"lora_alpha": 16}))
    if rank == 0:
        q.put([o.outputs[0].token_ids for o in outs])


def test_lora_tensor_parallel_matches_merged(tmp_path):
    """Column-parallel B rows and row-parallel A columns are cut like the base weights (Gloo, world size 2)."""
    import shutil

    import torch.multiprocessing as mp
    from safetensors.torch import load_file, save_file

    from vllm_metax_b200 import LLM, SamplingParams

    src = LLM(tiny_cfg(), **KW)
    d = str(tmp_path / "base")
    export_hf_checkpoint(src.engine.runner.model, d)
    base = load_file(os.path.join(d, "model.safetensors"))
    adapter = make_adapter(base, 8, 5)
    dm = str(tmp_path / "merged")
    os.makedirs(dm)
    save_file(merged(base, adapter, 16), os.path.join(dm, "model.safetensors"))
    shutil.copy(os.path.join(d, "config.json"), dm)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 45)]
    want = [o.outputs[0].token_ids for o in
            LLM(dm, dtype=torch.float32, **KW).generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29250 + os.getpid() % 40
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, d, adapter, prompts, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
