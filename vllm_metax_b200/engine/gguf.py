"""GGUF checkpoints (llama.cpp's single-file format): header / metadata / tensor-table parser, block de-quantisers and
the mapping onto this package's Llama-family loaders.

    LLM("/models/llama-3.1-8b-q4_k_m.gguf")        # config comes from the file's metadata

Tensors are de-quantised to the model dtype while loading (weight-only support: the file format and its block codes
are handled, the kernels then run in bf16).  Block codes: F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q4_K, Q6_K - the ones the
common Q8_0 / Q4_0 / Q4_K_M / Q6_K exports use.  For the ``llama`` architecture the q / k projection rows are stored
pairwise-interleaved per head (llama.cpp's rotary layout) and are put back to the half-split order.

Parity: ``gguf`` in the reference's list of supported quantisation methods (vllm_metax/platform.py:177-189), served
there by upstream's GGUF loader.
"""
from __future__ import annotations

import struct
from typing import Iterator

import numpy as np
import torch

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 3, 8, 12, 14, 30
# type -> (values per block, bytes per block)
BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20),
         GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos: self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, t: int):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF metadata type {t}")


def read_gguf(path: str):
    """-> ``(metadata dict, {name: (shape (outermost first), ggml type, absolute byte offset)}, memory map)``."""
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    r = _Reader(mm)
    if bytes(mm[:4]) != b"GGUF":
        raise ValueError(f"{path} is not a GGUF file")
    r.pos = 4
    version, n_tensors, n_kv = r.take("<I"), r.take("<Q"), r.take("<Q")
    if version < 2:
        raise ValueError(f"GGUF version {version} is not supported")
    meta = {}
    for _ in range(n_kv):
        key = r.string()
        meta[key] = r.value(r.take("<I"))
    infos = {}
    for _ in range(n_tensors):
        name = r.string()
        nd = r.take("<I")
        dims = [r.take("<Q") for _ in range(nd)]
        typ, off = r.take("<I"), r.take("<Q")
        infos[name] = (tuple(reversed(dims)), typ, off)
    align = int(meta.get("general.alignment", 32))
    base = (r.pos + align - 1) // align * align
    return meta, {k: (s, t, base + o) for k, (s, t, o) in infos.items()}, mm


def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.view(np.float16).astype(np.float32)


def dequantize(raw: np.ndarray, typ: int, n: int) -> np.ndarray:
    """``raw`` uint8 bytes of ``n`` values in ggml block code ``typ`` -> float32 ``[n]``."""
    if typ == GGML_F32:
        return raw.view(np.float32).copy()
    if typ == GGML_F16:
        return _f16(raw)
    if typ == GGML_BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    if typ not in BLOCK:
        raise NotImplementedError(f"ggml tensor type {typ} is not supported (F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q4_K, Q6_K are)")
    per, size = BLOCK[typ]
    b = raw.reshape(n // per, size)
    if typ == GGML_Q8_0:
        return (_f16(b[:, :2].copy()) * b[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if typ in (GGML_Q4_0, GGML_Q4_1):
        hdr = 2 if typ == GGML_Q4_0 else 4
        d = _f16(b[:, :2].copy())
        qs = b[:, hdr:]
        q = np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32)
        if typ == GGML_Q4_0:
            return (d * (q - 8.0)).reshape(-1)
        return (d * q + _f16(b[:, 2:4].copy())).reshape(-1)
    if typ == GGML_Q4_K:
        d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())            # [nb, 1]
        sc = b[:, 4:16]
        scale = np.empty((b.shape[0], 8), np.float32)
        mins = np.empty((b.shape[0], 8), np.float32)
        scale[:, :4], mins[:, :4] = sc[:, 0:4] & 63, sc[:, 4:8] & 63
        scale[:, 4:] = (sc[:, 8:12] & 0xF) | ((sc[:, 0:4] >> 6) << 4)
        mins[:, 4:] = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
        qs = b[:, 16:].reshape(-1, 4, 32)                                    # 4 groups of 64 values
        q = np.stack([qs & 0xF, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)
        return ((d * scale)[:, :, None] * q - (dmin * mins)[:, :, None]).reshape(-1)
    # Q6_K
    ql, qh = b[:, :128].reshape(-1, 2, 64), b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = _f16(b[:, 208:210].copy())
    lo, hi = ql[:, :, :32], ql[:, :, 32:]
    q = np.stack([(lo & 0xF) | ((qh & 3) << 4), (hi & 0xF) | (((qh >> 2) & 3) << 4),
                  (lo >> 4) | (((qh >> 4) & 3) << 4), (hi >> 4) | (((qh >> 6) & 3) << 4)], 2)      # [nb, 2, 4, 32]
    q = q.astype(np.float32) - 32.0
    s = sc.reshape(-1, 2, 4, 2)                                              # scale index = 2 * quarter + l // 16
    s = np.repeat(s, 16, axis=3)
    return (d[:, :, None, None] * s * q).reshape(-1)


_NAMES = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}
_LAYER = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
          "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
          "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
          "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm"}
_ARCH = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "mistral": "MistralForCausalLM"}


def hf_name(name: str):
    stem, _, kind = name.rpartition(".")
    if stem in _NAMES:
        return f"{_NAMES[stem]}.{kind}"
    parts = stem.split(".")
    if len(parts) == 3 and parts[0] == "blk" and parts[2] in _LAYER:
        return f"model.layers.{parts[1]}.{_LAYER[parts[2]]}.{kind}"
    return None


def config_from_gguf(meta: dict, infos: dict) -> dict:
    """The file's metadata as a Hugging Face style ``config.json`` dict."""
    arch = meta.get("general.architecture", "llama")
    if arch not in _ARCH:
        raise NotImplementedError(f"GGUF architecture {arch!r} is not mapped (known: {sorted(_ARCH)})")
    g = lambda k, default=None: meta.get(f"{arch}.{k}", default)
    heads = int(g("attention.head_count"))
    hidden = int(g("embedding_length"))
    cfg = {"architectures": [_ARCH[arch]], "hidden_size": hidden, "num_hidden_layers": int(g("block_count")),
           "intermediate_size": int(g("feed_forward_length")), "num_attention_heads": heads,
           "num_key_value_heads": int(g("attention.head_count_kv", heads)),
           "head_dim": int(g("attention.key_length", hidden // heads)),
           "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)), "rope_theta": float(g("rope.freq_base", 10000.0)),
           "max_position_embeddings": int(g("context_length", 4096)),
           "vocab_size": int(g("vocab_size", infos["token_embd.weight"][0][0])),
           "tie_word_embeddings": "output.weight" not in infos}
    for key, name in (("tokenizer.ggml.eos_token_id", "eos_token_id"), ("tokenizer.ggml.bos_token_id", "bos_token_id")):
        if key in meta:
            cfg[name] = int(meta[key])
    return cfg


def iter_gguf(path: str, dtype=torch.bfloat16) -> Iterator[tuple[str, torch.Tensor]]:
    """``(HF tensor name, tensor)`` pairs with every block code expanded to ``dtype``."""
    meta, infos, mm = read_gguf(path)
    arch = meta.get("general.architecture", "llama")
    heads = int(meta.get(f"{arch}.attention.head_count", 1))
    kv = int(meta.get(f"{arch}.attention.head_count_kv", heads))
    for name, (shape, typ, off) in infos.items():
        target = hf_name(name)
        if target is None:
            continue
        n = int(np.prod(shape))
        per, size = BLOCK.get(typ, (1, 0))
        if size == 0:
            dequantize(np.zeros(0, np.uint8), typ, 0)        # raises with the unsupported-type message
        w = torch.from_numpy(dequantize(np.asarray(mm[off: off + n // per * size]), typ, n).reshape(shape))
        if arch == "llama" and (".q_proj.weight" in target or ".k_proj.weight" in target):
            h = heads if ".q_proj." in target else kv           # rows (r0 i0 r1 i1 ...) per head -> (r0 r1 ... i0 i1 ...)
            w = w.reshape(h, shape[0] // h // 2, 2, *shape[1:]).transpose(1, 2).reshape(shape)
        yield target, w.to(dtype)
