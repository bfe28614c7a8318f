"""GGUF single-file checkpoints: block de-quantisers against scalar re-statements of the ggml block layouts, the file
parser, and a Llama checkpoint written as GGUF (with llama.cpp's q / k row interleave) against Hugging Face."""
import struct

import numpy as np
import pytest
import torch

from vllm_metax_b200.engine import gguf as G


def _f16(b):
    return float(np.frombuffer(bytes(b), np.float16)[0])


def _scalar_q4_k(block):
    block = [int(x) for x in block]
    d, dmin, sc, qs = _f16(block[0:2]), _f16(block[2:4]), block[4:16], block[16:144]
    out, qi, isub = [], 0, 0

    def scale_min(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)

    for _ in range(4):
        s1, m1 = scale_min(isub)
        s2, m2 = scale_min(isub + 1)
        out += [d * s1 * (qs[qi + l] & 0xF) - dmin * m1 for l in range(32)]
        out += [d * s2 * (qs[qi + l] >> 4) - dmin * m2 for l in range(32)]
        qi += 32
        isub += 2
    return out


def _scalar_q6_k(block):
    block = [int(x) for x in block]                     # python ints: the "- 32" must not wrap
    ql, qh = block[0:128], block[128:192]
    sc = np.frombuffer(bytes(block[192:208]), np.int8)
    d = _f16(block[208:210])
    y = [0.0] * 256
    for half in range(2):
        for l in range(32):
            i = l // 16
            a, b_, h = ql[64 * half + l], ql[64 * half + l + 32], qh[32 * half + l]
            q1 = ((a & 0xF) | ((h & 3) << 4)) - 32
            q2 = ((b_ & 0xF) | (((h >> 2) & 3) << 4)) - 32
            q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32
            q4 = ((b_ >> 4) | (((h >> 6) & 3) << 4)) - 32
            o = 128 * half
            y[o + l] = d * sc[8 * half + i] * q1
            y[o + l + 32] = d * sc[8 * half + i + 2] * q2
            y[o + l + 64] = d * sc[8 * half + i + 4] * q3
            y[o + l + 96] = d * sc[8 * half + i + 6] * q4
    return y


def _random_blocks(typ, nb, rng):
    per, size = G.BLOCK[typ]
    raw = rng.integers(0, 256, (nb, size), dtype=np.uint8)
    halves = {G.GGML_Q4_K: [(0, 2), (2, 4)], G.GGML_Q6_K: [(208, 210)], G.GGML_Q8_0: [(0, 2)], G.GGML_Q4_0: [(0, 2)],
              G.GGML_Q4_1: [(0, 2), (2, 4)]}[typ]
    for lo, hi in halves:                                   # finite, small scales
        raw[:, lo:hi] = rng.uniform(0.01, 0.1, (nb, 1)).astype(np.float16).view(np.uint8)
    return raw


def test_block_codes_match_scalar_statements():
    rng = np.random.default_rng(0)
    raw = _random_blocks(G.GGML_Q4_K, 3, rng)
    got = G.dequantize(raw.reshape(-1), G.GGML_Q4_K, 3 * 256)
    np.testing.assert_allclose(got, np.concatenate([_scalar_q4_k(b) for b in raw]), rtol=1e-5, atol=1e-6)
    raw = _random_blocks(G.GGML_Q6_K, 3, rng)
    got = G.dequantize(raw.reshape(-1), G.GGML_Q6_K, 3 * 256)
    np.testing.assert_allclose(got, np.concatenate([_scalar_q6_k(b) for b in raw]), rtol=1e-5, atol=1e-6)
    raw = _random_blocks(G.GGML_Q8_0, 2, rng)
    want = np.concatenate([_f16(b[:2]) * np.frombuffer(bytes(b[2:]), np.int8).astype(np.float32) for b in raw])
    np.testing.assert_allclose(G.dequantize(raw.reshape(-1), G.GGML_Q8_0, 64), want, rtol=1e-6)
    raw = _random_blocks(G.GGML_Q4_0, 2, rng)
    want = np.concatenate([_f16(b[:2]) * (np.concatenate([b[2:] & 0xF, b[2:] >> 4]).astype(np.float32) - 8) for b in raw])
    np.testing.assert_allclose(G.dequantize(raw.reshape(-1), G.GGML_Q4_0, 64), want, rtol=1e-6)
    raw = _random_blocks(G.GGML_Q4_1, 2, rng)
    want = np.concatenate([_f16(b[:2]) * np.concatenate([b[4:] & 0xF, b[4:] >> 4]).astype(np.float32) + _f16(b[2:4]) for b in raw])
    np.testing.assert_allclose(G.dequantize(raw.reshape(-1), G.GGML_Q4_1, 64), want, rtol=1e-6)
    with pytest.raises(NotImplementedError):
        G.dequantize(np.zeros(0, np.uint8), 13, 0)


def _q8_0(w):
    b = w.reshape(-1, 32)
    d = np.abs(b).max(1, keepdims=True) / 127.0
    d = np.maximum(d, 1e-8).astype(np.float16)
    q = np.clip(np.round(b / d.astype(np.float32)), -127, 127).astype(np.int8)
    return np.concatenate([d.view(np.uint8), q.view(np.uint8)], 1).reshape(-1), (d.astype(np.float32) * q).reshape(w.shape)


def _write_gguf(path, meta, tensors):
    """``tensors``: {name: (shape outermost-first, ggml type, raw bytes)}."""
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        out += s(k)
        if isinstance(v, str):
            out += struct.pack("<I", 8) + s(v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        else:
            out += struct.pack("<II", 4, v)
    off, blobs = 0, []
    for name, (shape, typ, raw) in tensors.items():
        out += s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        out += struct.pack("<IQ", typ, off)
        pad = (-len(raw)) % 32
        blobs.append(bytes(raw) + bytes(pad))
        off += len(raw) + pad
    out += bytes((-len(out)) % 32)
    with open(path, "wb") as f:
        f.write(out + b"".join(blobs))


def test_llama_gguf_file_matches_hugging_face(tmp_path):
    tf = pytest.importorskip("transformers")
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    H, Hkv, D = 4, 2, 32
    hf = tf.LlamaForCausalLM(tf.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                            num_attention_heads=H, num_key_value_heads=Hkv, max_position_embeddings=256)).eval().float()
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    layer = {v: k for k, v in G._LAYER.items()}
    tensors = {}
    with torch.no_grad():
        for name, p in hf.named_parameters():
            w = p.detach().clone()
            if name in names:
                gname = names[name]
            else:
                parts = name.split(".")
                gname = f"blk.{parts[2]}.{layer['.'.join(parts[3:-1])]}.{parts[-1]}"
            if ".q_proj." in name or ".k_proj." in name:           # llama.cpp stores rotary pairs side by side
                h = H if ".q_proj." in name else Hkv
                w = w.reshape(h, 2, w.shape[0] // h // 2, w.shape[1]).transpose(1, 2).reshape(w.shape)
            arr = w.numpy()
            if w.dim() == 2 and "embd" not in gname:                # matrices as Q8_0; write the rounded values back
                raw, back = _q8_0(arr)
                tensors[gname] = (tuple(arr.shape), G.GGML_Q8_0, raw)
                if ".q_proj." in name or ".k_proj." in name:
                    h = H if ".q_proj." in name else Hkv
                    back = torch.from_numpy(back).reshape(h, back.shape[0] // h // 2, 2, back.shape[1]).transpose(1, 2).reshape(back.shape).numpy()
                p.copy_(torch.from_numpy(np.ascontiguousarray(back)))
            else:
                tensors[gname] = (tuple(arr.shape), G.GGML_F32, arr.astype(np.float32).tobytes())
    meta = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 128,
            "llama.feed_forward_length": 256, "llama.attention.head_count": H, "llama.attention.head_count_kv": Hkv,
            "llama.attention.layer_norm_rms_epsilon": float(hf.config.rms_norm_eps), "llama.rope.freq_base": 10000.0,
            "llama.context_length": 256}
    path = str(tmp_path / "tiny.gguf")
    _write_gguf(path, meta, {k: (s_, t, np.frombuffer(r, np.uint8) if isinstance(r, bytes) else r) for k, (s_, t, r) in tensors.items()})
    m, infos, _ = G.read_gguf(path)
    assert m["llama.block_count"] == 2 and infos["blk.0.attn_q.weight"][0] == (128, 128)
    llm = LLM(path, dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=16, block_size=16)
    ids = [[5, 9, 33, 100, 7, 8, 200, 31, 2, 17, 45], [3, 4, 5, 6]]
    outs = llm.generate(ids, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    got_h = llm.embed(ids, pooling="mean", normalize=False)
    for i, p in enumerate(ids):
        with torch.no_grad():
            t = torch.tensor([p])
            want = hf.generate(t, max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(p):].tolist()
            want_h = hf.base_model(t).last_hidden_state[0].mean(0)
        assert list(outs[i].outputs[0].token_ids) == want
        torch.testing.assert_close(got_h[i], want_h, atol=2e-4, rtol=2e-4)
