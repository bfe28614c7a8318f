"""The ``torch.ops._C`` / ``torch.ops._C_cache_ops`` names upstream vLLM layers bind to, implemented on this package's
kernels.

Upstream layers look their kernels up by name when they are constructed (``SiluAndMul.__init__`` reads
``torch.ops._C.silu_and_mul``) or through ``vllm._custom_ops`` wrappers.  A platform plugin ships those names itself:
the reference builds a ``_C`` extension with the upstream schemas from its own sources
(csrc/libtorch_stable/torch_bindings.cpp:31-742, csrc/cache_kernels.cu); here they are thin ``torch.library``
definitions over ``torch.ops.b200``.  A name that already exists (an upstream ``vllm._C`` loaded in the same
process) is left alone.
"""
from __future__ import annotations

import torch

from .. import _custom_ops as ops

_LIBS: list = []
DEFINED: list[str] = []


def _has(ns: str, name: str) -> bool:
    try:
        getattr(getattr(torch.ops, ns), name)
        return True
    except (AttributeError, RuntimeError):
        return False


def _define(lib, ns: str, schema: str, fn) -> None:
    name = schema.split("(")[0]
    if _has(ns, name):
        return
    lib.define(schema)
    lib.impl(name, fn, "CUDA")
    DEFINED.append(f"{ns}::{name}")


def _act(name: str, p0_from=None):
    def fn(out, x, *extra):
        p0 = float(extra[0]) if len(extra) > 0 else 0.0
        p1 = float(extra[1]) if len(extra) > 1 else 0.0
        ops.act_and_mul(x, name, out=out, p0=p0, p1=p1)

    return fn


def _unary(name: str):
    def fn(out, x):
        out.copy_(ops.activation(x, name))

    return fn


def _rms_norm(out, x, weight, eps):
    ops.rms_norm(x.reshape(-1, x.shape[-1]), weight, float(eps), out=out.view(-1, x.shape[-1]))


def _fused_add_rms_norm(x, residual, weight, eps):
    ops.fused_add_rms_norm(x.view(-1, x.shape[-1]), residual.view(-1, x.shape[-1]), weight, float(eps))


_cs_cache: dict = {}


def fp32_cos_sin(cache: torch.Tensor) -> torch.Tensor:
    """The rotary table in fp32 (the kernels' table type), converted once per table."""
    if cache.dtype == torch.float32:
        return cache
    key = (cache.data_ptr(), tuple(cache.shape), cache.dtype)
    got = _cs_cache.get(key)
    if got is None:
        got = cache.float().contiguous()
        _cs_cache[key] = got
    return got


def _rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox):
    T = positions.numel()
    q2 = query.view(T, -1)
    k2 = key.view(T, -1) if key is not None else None
    ops.rotary_embedding(positions.reshape(-1), q2, k2, int(head_size), fp32_cos_sin(cos_sin_cache), bool(is_neox))


def _reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale):
    # upstream passes the two halves of one [blocks, 2, block_size, heads, dim] allocation as views
    raise NotImplementedError("this platform's attention backend writes the cache itself")


def _apply_repetition_penalties(logits, prompt_mask, output_mask, repetition_penalties):
    pen = torch.where(prompt_mask | output_mask, repetition_penalties.unsqueeze(1).to(logits.dtype),
                      torch.ones((), dtype=logits.dtype, device=logits.device))
    logits.mul_(torch.where(logits > 0, 1.0 / pen, pen))


def _topk(scoring: str):
    def fn(topk_weights, topk_ids, token_expert_indices, gating_output, renormalize=False, bias=None):
        T, k = topk_weights.shape
        w, ids = ops.topk_gating(gating_output.reshape(T, -1), k, bool(renormalize), scoring,
                                 None if bias is None else bias.float())
        topk_weights.copy_(w)
        topk_ids.copy_(ids)
        if token_expert_indices is not None and token_expert_indices.numel():
            # the position of every (token, choice) pair in choice-major order, as upstream's kernel fills it
            token_expert_indices.copy_(torch.arange(k, device=ids.device, dtype=token_expert_indices.dtype)[None, :] * T
                                       + torch.arange(T, device=ids.device, dtype=token_expert_indices.dtype)[:, None])

    return fn


def _grouped_topk(scores, num_expert_group, topk_group, topk, renormalize, routed_scaling_factor, bias, scoring_func=0):
    if int(scoring_func) == 1:      # `scores` are logits: sigmoid + bias + group-limited top-k in one kernel
        return ops.grouped_topk(scores, int(topk), bool(renormalize), int(num_expert_group), int(topk_group),
                                "sigmoid", bias, float(routed_scaling_factor))
    # already-activated scores: the same selection in tensor ops (bias steers the choice, not the weights)
    T, E = scores.shape
    sc = scores.float()
    choice = sc + bias.float()[None, :]
    grp = choice.view(T, num_expert_group, -1)
    gscore = grp.topk(2, dim=-1).values.sum(-1) if grp.shape[-1] >= 2 else grp.max(-1).values
    gidx = gscore.topk(topk_group, dim=-1).indices
    gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
    mask = gmask[:, :, None].expand_as(grp).reshape(T, E)
    ids = choice.masked_fill(mask == 0, float("-inf")).topk(topk, dim=-1).indices
    w = sc.gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * float(routed_scaling_factor), ids.to(torch.int32)


def _moe_sum(inp, out):
    torch.sum(inp, dim=1, out=out)


def define_c_ops() -> list[str]:
    """Define the missing names (idempotent).  Returns the fully qualified names this call or an earlier one defined."""
    if _LIBS:
        return DEFINED
    lib = torch.library.Library("_C", "FRAGMENT")
    _LIBS.append(lib)
    for op, act in (("silu_and_mul", "silu"), ("mul_and_silu", "mul_silu"), ("gelu_and_mul", "gelu"),
                    ("gelu_tanh_and_mul", "gelu_tanh")):
        _define(lib, "_C", f"{op}(Tensor! result, Tensor input) -> ()", _act(act))
    _define(lib, "_C", "fatrelu_and_mul(Tensor! result, Tensor input, float threshold) -> ()", _act("fatrelu"))
    _define(lib, "_C", "swigluoai_and_mul(Tensor! result, Tensor input, float alpha=1.702, float limit=7.0) -> ()",
            _act("swigluoai"))
    _define(lib, "_C", "silu_and_mul_with_clamp(Tensor! result, Tensor input, float limit) -> ()",
            lambda out, x, limit: ops.act_and_mul(x, "swiglustep", out=out, p1=float(limit)))
    for op in ("gelu_new", "gelu_fast", "gelu_quick"):
        _define(lib, "_C", f"{op}(Tensor! out, Tensor input) -> ()", _unary(op))
    _define(lib, "_C", "activation_lut_bf16(Tensor! out, Tensor input, Tensor lut) -> ()",
            lambda out, x, lut: out.copy_(lut[x.view(torch.int16).to(torch.int32) & 0xFFFF].view_as(x)))
    _define(lib, "_C", "rms_norm(Tensor! result, Tensor input, Tensor weight, float epsilon) -> ()", _rms_norm)
    _define(lib, "_C", "fused_add_rms_norm(Tensor! input, Tensor! residual, Tensor weight, float epsilon) -> ()",
            _fused_add_rms_norm)
    _define(lib, "_C", "rotary_embedding(Tensor positions, Tensor! query, Tensor!? key, int head_size, "
            "Tensor cos_sin_cache, bool is_neox) -> ()", _rotary_embedding)
    _define(lib, "_C", "apply_repetition_penalties_(Tensor! logits, Tensor prompt_mask, Tensor output_mask, "
            "Tensor repetition_penalties) -> ()", _apply_repetition_penalties)
    _define(lib, "_C", "weak_ref_tensor(Tensor input) -> Tensor", lambda t: torch.ops.b200.weak_ref_tensor(t))
    # routing ops of the MoE namespace (upstream's router calls them by name)
    moe = torch.library.Library("_moe_C", "FRAGMENT")
    _LIBS.append(moe)
    for op, scoring in (("topk_softmax", "softmax"), ("topk_sigmoid", "sigmoid")):
        _define(moe, "_moe_C", f"{op}(Tensor! topk_weights, Tensor! topk_indices, Tensor! token_expert_indices, "
                "Tensor gating_output, bool renormalize, Tensor? bias) -> ()", _topk(scoring))
    _define(moe, "_moe_C", "grouped_topk(Tensor scores, int n_group, int topk_group, int topk, bool renormalize, "
            "float routed_scaling_factor, Tensor bias, int scoring_func) -> (Tensor, Tensor)", _grouped_topk)
    _define(moe, "_moe_C", "moe_sum(Tensor input, Tensor! output) -> ()", _moe_sum)
    return DEFINED
