"""The package as a vLLM platform plugin, live: upstream ``vllm.LLM`` discovers the three entry points, resolves
``B200Platform``, builds its engine on this package's attention backend and kernels, and generates.  The tokens are
compared with the standalone engine on the same checkpoint.

vLLM runs in a child process (it owns global state: the current platform, custom-op registries, the CUDA
allocator); the entry points are supplied through a ``.dist-info`` folder on ``PYTHONPATH``, which is what a
``pip install`` of the package would write.
"""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytest.importorskip("vllm")
tf = pytest.importorskip("transformers")


def write_dist_info(folder: str) -> None:
    d = os.path.join(folder, "vllm_metax_b200-0.0.0.dist-info")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "METADATA"), "w") as f:
        f.write("Metadata-Version: 2.1\nName: vllm_metax_b200\nVersion: 0.0.0\n")
    with open(os.path.join(d, "entry_points.txt"), "w") as f:
        f.write(textwrap.dedent("""\
            [vllm.platform_plugins]
            b200 = vllm_metax_b200:register

            [vllm.general_plugins]
            b200_out_of_tree = vllm_metax_b200:register_out_of_tree
            b200_models = vllm_metax_b200:register_model
            """))


CHILD = r"""
import json, os, sys
import torch
from vllm import LLM, SamplingParams
from vllm.platforms import current_platform
path, out, eager = sys.argv[1], sys.argv[2], sys.argv[3] == "1"
prompts = json.load(open(os.path.join(path, "prompts.json")))
llm = LLM(path, dtype="bfloat16", max_model_len=512, gpu_memory_utilization=0.25, enforce_eager=eager,
          max_num_seqs=8, seed=0)
outs = llm.generate([{"prompt_token_ids": p} for p in prompts], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
from vllm_metax_b200 import _custom_ops as ops
from vllm.model_executor.custom_op import op_registry_oot
moe = op_registry_oot.get("UnquantizedFusedMoEMethod")
res = {"platform": type(current_platform).__name__, "module": type(current_platform).__module__,
       "tokens": [list(o.outputs[0].token_ids) for o in outs], "launches": ops.launch_count(),
       "moe_method": moe.__name__ if moe is not None else ""}
json.dump(res, open(out, "w"))
"""


def _checkpoint(path: str, kind: str) -> list:
    torch.manual_seed(0)
    if kind == "llama":
        cfg = tf.LlamaConfig(vocab_size=2048, hidden_size=1024, intermediate_size=2816, num_hidden_layers=3,
                             num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024,
                             rms_norm_eps=1e-5, tie_word_embeddings=False)
        tf.LlamaForCausalLM(cfg).save_pretrained(path)
    elif kind == "qwen3_moe":
        cfg = tf.Qwen3MoeConfig(vocab_size=2048, hidden_size=1024, intermediate_size=2048, num_hidden_layers=2,
                                num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024,
                                rms_norm_eps=1e-6, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                                moe_intermediate_size=512, decoder_sparse_step=1, norm_topk_prob=True, mlp_only_layers=[])
        tf.Qwen3MoeForCausalLM(cfg).save_pretrained(path)
    else:
        raise ValueError(kind)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (100, 33, 200)]
    json.dump(prompts, open(os.path.join(path, "prompts.json"), "w"))
    return prompts


def _standalone_tokens(path: str, prompts: list) -> list:
    from vllm_metax_b200 import LLM, SamplingParams

    llm = LLM(path, device="cuda", dtype="bfloat16", block_size=64, max_model_len=512, max_num_seqs=8,
              max_num_batched_tokens=1024, num_gpu_blocks=128)
    toks = [list(o.outputs[0].token_ids) for o in llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
    llm.engine.runner.graphs.clear()
    del llm
    torch.cuda.empty_cache()
    return toks


def run_vllm_child(path: str, eager: bool, log_path: str | None = None) -> dict:
    write_dist_info(path)
    out = os.path.join(path, "vllm_out.json")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([path, ROOT, env.get("PYTHONPATH", "")])
    env.update(VLLM_PLUGINS="b200,b200_out_of_tree,b200_models", VLLM_ENABLE_V1_MULTIPROCESSING="0",
               VLLM_LOGGING_LEVEL="INFO", TOKENIZERS_PARALLELISM="false")
    script = os.path.join(path, "child.py")
    with open(script, "w") as f:
        f.write(CHILD)
    r = subprocess.run([sys.executable, script, path, out, "1" if eager else "0"], env=env, capture_output=True,
                       text=True, timeout=900)
    if log_path:
        with open(log_path, "w") as f:
            f.write(r.stdout[-20000:] + "\n==== stderr ====\n" + r.stderr[-40000:])
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-6000:])
    return json.load(open(out))


@pytest.mark.parametrize("eager", [True, False])
def test_vllm_llm_generate_on_b200_platform(tmp_path, eager):
    path = str(tmp_path)
    prompts = _checkpoint(path, "llama")
    want = _standalone_tokens(path, prompts)
    got = run_vllm_child(path, eager, os.environ.get("B200_VLLM_LIVE_LOG"))
    assert got["platform"].endswith("B200Platform") and got["module"] == "vllm_metax_b200.platform", got
    assert got["launches"] > 0, "no kernel of this package ran under vLLM"
    toks = got["tokens"]
    assert [t[0] for t in toks] == [w[0] for w in want], (toks, want)
    prefix = [next((i for i, (a, b) in enumerate(zip(t, w)) if a != b), len(w)) for t, w in zip(toks, want)]
    assert min(prefix) >= 2 and sum(prefix) >= 3 * len(want), (prefix, toks, want)


def test_vllm_moe_runs_on_grouped_gemms(tmp_path):
    """A Qwen3-MoE checkpoint under upstream vLLM: the experts run through this package's FusedMoE method."""
    path = str(tmp_path)
    prompts = _checkpoint(path, "qwen3_moe")
    want = _standalone_tokens(path, prompts)
    got = run_vllm_child(path, True, os.environ.get("B200_VLLM_LIVE_LOG"))
    assert got["platform"].endswith("B200Platform"), got
    assert got.get("moe_method", "").startswith("B200"), got
    toks = got["tokens"]
    assert [t[0] for t in toks] == [w[0] for w in want], (toks, want)
    prefix = [next((i for i, (a, b) in enumerate(zip(t, w)) if a != b), len(w)) for t, w in zip(toks, want)]
    assert min(prefix) >= 2 and sum(prefix) >= 3 * len(want), (prefix, toks, want)


def _tokenizer(path: str) -> None:
    """A word-level tokenizer over the checkpoint's 2048 ids with a trivial chat template (no download needed)."""
    tokenizers = pytest.importorskip("tokenizers")
    vocab = {f"w{i}": i for i in range(2048)}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    fast = tf.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="w0", eos_token="w1", bos_token="w2", pad_token="w3")
    fast.chat_template = "{% for m in messages %}{{ m['content'] }} {% endfor %}"
    fast.save_pretrained(path)


def test_vllm_serve_chat_round_trip(tmp_path):
    """``vllm serve`` on the plugin platform answers one /v1/chat/completions request."""
    import socket
    import time
    import urllib.request

    path = str(tmp_path)
    _checkpoint(path, "llama")
    _tokenizer(path)
    write_dist_info(path)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([path, ROOT, env.get("PYTHONPATH", "")])
    env.update(VLLM_PLUGINS="b200,b200_out_of_tree,b200_models", VLLM_LOGGING_LEVEL="INFO", TOKENIZERS_PARALLELISM="false")
    log = open(os.path.join(path, "serve.log"), "w")
    proc = subprocess.Popen([sys.executable, "-m", "vllm.entrypoints.openai.api_server", "--model", path,
                             "--served-model-name", "tiny", "--dtype", "bfloat16", "--max-model-len", "512",
                             "--gpu-memory-utilization", "0.25", "--host", "127.0.0.1", "--port", str(port),
                             "--max-num-seqs", "8"], env=env, stdout=log, stderr=subprocess.STDOUT)
    try:
        deadline = time.time() + 600
        up = False
        while time.time() < deadline and proc.poll() is None:
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2)
                up = True
                break
            except Exception:
                time.sleep(2)
        assert up, open(os.path.join(path, "serve.log")).read()[-6000:]
        body = json.dumps({"model": "tiny", "messages": [{"role": "user", "content": "w5 w17 w200 w33"}],
                           "max_tokens": 8, "temperature": 0}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        resp = json.loads(urllib.request.urlopen(req, timeout=120).read())
        assert resp["choices"][0]["message"]["content"] is not None
        assert resp["usage"]["completion_tokens"] == 8
        record = os.environ.get("B200_VLLM_LIVE_LOG")
        if record:
            with open(record + ".serve.json", "w") as f:
                json.dump(resp, f, indent=1)
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
        log.close()
        record = os.environ.get("B200_VLLM_LIVE_LOG")
        if record:
            with open(record + ".serve.log", "w") as f:
                f.write(open(os.path.join(path, "serve.log")).read()[-30000:])
