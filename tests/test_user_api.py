"""User-level API beyond generate: chat, embeddings / scores / zero-shot classification, constrained decoding,
weight updates (the features the reference's shipped examples exercise)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=32, num_gpu_blocks=64)


@pytest.fixture(scope="module")
def llm():
    from vllm_metax_b200 import LLM

    return LLM(tiny_cfg(), **KW)


def test_token_trie():
    from vllm_metax_b200.engine.structured import TokenTrie

    t = TokenTrie([[5, 6], [5, 7, 8], [9]])
    assert sorted(t.allowed_after([])) == [5, 9]
    assert sorted(t.allowed_after([5])) == [6, 7]
    assert t.allowed_after([5, 6]) == [] and t.complete([5, 6]) and not t.complete([5, 7])
    assert t.complete([1])                     # left the trie: nothing more to generate
    with pytest.raises(ValueError):
        TokenTrie([])


def test_guided_choice_and_allowed_tokens(llm):
    from vllm_metax_b200 import SamplingParams

    choices = [[11, 12, 13], [11, 40], [77]]
    prompts = [[1, 2, 3, 4], [9, 8, 7], [5] * 40]
    for temp in (0.0, 1.0):
        outs = llm.generate(prompts, SamplingParams(max_tokens=10, temperature=temp, seed=3, guided_choice=choices))
        for o in outs:
            assert o.outputs[0].token_ids in choices
            assert o.outputs[0].finish_reason == "stop"
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True, allowed_token_ids=[3, 4, 5]))
    assert all(set(o.outputs[0].token_ids) <= {3, 4, 5} and len(o.outputs[0].token_ids) == 6 for o in outs)
    # a large bias on one token wins the arg-max
    outs = llm.generate(prompts[:1], SamplingParams(max_tokens=3, ignore_eos=True, logit_bias={123: 1e4}))
    assert outs[0].outputs[0].token_ids == [123, 123, 123]
    with pytest.raises(ValueError):                       # text-level guidance needs a tokenizer
        llm.generate(prompts[:1], SamplingParams(guided_regex="a+"))


def test_embed_score_classify(llm):
    g = torch.Generator().manual_seed(0)
    p = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (7, 50, 21)]      # 50 > 32: two prefill chunks
    e_last = llm.embed(p)
    e_mean = llm.embed(p, pooling="mean", normalize=False)
    assert e_last.shape == (3, 256) and e_mean.shape == (3, 256)
    torch.testing.assert_close(e_last.norm(dim=-1), torch.ones(3), rtol=1e-4, atol=1e-4)
    # one prompt at a time gives the same vectors as the batch (chunking and batching do not leak)
    torch.testing.assert_close(llm.embed([p[1]])[0], e_last[1], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(llm.embed([p[1]], pooling="mean", normalize=False)[0], e_mean[1], rtol=1e-4, atol=1e-4)
    s = llm.score(p[0], p)
    assert abs(s[0] - 1.0) < 1e-4 and all(-1.0001 <= x <= 1.0001 for x in s)
    probs = llm.classify(p, [10, 20, 30])
    assert probs.shape == (3, 3)
    torch.testing.assert_close(probs.sum(-1), torch.ones(3), rtol=1e-5, atol=1e-5)
    # consistent with what greedy decoding restricted to the classes picks
    from vllm_metax_b200 import SamplingParams

    outs = llm.generate(p, SamplingParams(max_tokens=1, allowed_token_ids=[10, 20, 30], ignore_eos=True))
    assert [o.outputs[0].token_ids[0] for o in outs] == [[10, 20, 30][i] for i in probs.argmax(-1).tolist()]


def test_update_weights_changes_outputs_and_resets_prefix_cache(tmp_path):
    from safetensors.torch import load_file, save_file

    from tests.test_tp_cpu import export_hf_checkpoint  # the HF-named view of a model's weights
    from vllm_metax_b200 import LLM, SamplingParams

    llm = LLM(tiny_cfg(), enable_prefix_caching=True, **KW)
    prompt = list(range(1, 40))
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    before = llm.generate([prompt], sp)[0].outputs[0].token_ids
    d = str(tmp_path / "ckpt")
    export_hf_checkpoint(llm.engine.runner.model, d)
    named = load_file(os.path.join(d, "model.safetensors"))
    g = torch.Generator().manual_seed(9)
    named = {k: v + 0.05 * torch.randn(v.shape, generator=g) for k, v in named.items()}      # "one optimiser step"
    save_file(named, os.path.join(d, "model.safetensors"))
    want = LLM(d, dtype=torch.float32, **KW).generate([prompt], sp)[0].outputs[0].token_ids
    assert llm.update_weights(named) == len(named)
    after = llm.generate([prompt], sp)[0].outputs[0].token_ids      # same prompt: a stale prefix hit would show here
    assert after == want
    assert after != before


def test_chat_builds_a_prompt(llm):
    class Tok:
        chat_template = None

        def encode(self, text, add_special_tokens=True):
            return [min(1023, ord(c)) for c in text]

        def decode(self, ids, **kw):
            return "".join(chr(i) for i in ids)

    from vllm_metax_b200 import SamplingParams

    llm.tokenizer = Tok()
    try:
        out = llm.chat([{"role": "user", "content": "hi"}], SamplingParams(max_tokens=2, ignore_eos=True))
        assert out[0].prompt == "user: hi\nassistant:" and len(out[0].outputs[0].token_ids) == 2
    finally:
        llm.tokenizer = None


def test_environment_switches(tmp_path, monkeypatch):
    """The switches of envs.py that act outside the kernels: the precision-dump directory makes every engine record
    its module outputs, the build target can be 'empty', the grouped top-k switch selects the unfused statement."""
    import json as _json

    from vllm_metax_b200 import LLM, SamplingParams, _build, envs
    from vllm_metax_b200.utils.precision_dump import load_dump

    monkeypatch.setenv("B200_PRECISION_DUMP_DIR", str(tmp_path))
    assert envs.B200_PRECISION_DUMP_DIR == str(tmp_path)
    from tests.test_e2e_plumbing import tiny_cfg

    llm = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=64, max_num_seqs=2, max_num_batched_tokens=32,
              num_gpu_blocks=16)
    llm.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=2))
    llm._precision_dump.__exit__()
    recs = load_dump(str(tmp_path / "dump_rank0.jsonl"))
    assert len(recs) > 10 and any("layers" in k[0] for k in recs)
    monkeypatch.setenv("B200_TARGET_DEVICE", "empty")
    assert _build.build() is None
    monkeypatch.setenv("B200_USE_FUSED_GROUPED_TOPK", "0")
    assert not envs.B200_USE_FUSED_GROUPED_TOPK


def test_batch_invariant_switch_pins_the_batch_dependent_choices():
    """B200_BATCH_INVARIANT=1 (checked in a fresh interpreter: the switch is read once): unsplit decode attention, the
    native GEMM dispatcher's split-K / stream-K / pair switches off, cascade attention and fused collectives off; and
    a request generates the same tokens alone and inside a batch."""
    import subprocess
    import sys

    code = '''
import os, json, torch
import vllm_metax_b200 as pkg
from vllm_metax_b200 import _custom_ops as ops, LLM, SamplingParams
from tests.test_e2e_plumbing import tiny_cfg
assert ops.batch_invariant()
assert ops.decode_num_splits(1, 1, 100000) == 1 and ops.decode_num_splits(3, 8, 4096) == 1
assert all(os.environ[k] == "0" for k in ("B200_GEMM_STREAMK", "B200_GEMM_SPLITK", "B200_GEMM_PAIR",
                                          "B200_FUSED_TP_COLLECTIVES", "B200_CASCADE_ATTENTION", "B200_CUSTOM_ALLREDUCE"))
llm = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)
g = torch.Generator().manual_seed(0)
prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (30, 9, 50, 17)]
sp = SamplingParams(max_tokens=6, ignore_eos=True)
alone = [llm.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
together = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
print("RESULT", json.dumps(alone == together))
'''
    env = dict(os.environ, B200_BATCH_INVARIANT="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, env=env, timeout=300)
    assert r.returncode == 0 and "RESULT true" in r.stdout, (r.stdout[-500:], r.stderr[-1500:])
    from vllm_metax_b200 import _custom_ops as ops

    assert not ops.batch_invariant() and ops.decode_num_splits(1, 1, 100000) > 1       # off by default
