"""Constrained decoding: the sampler masks the logits of a request down to the tokens its constraint allows.

* ``allowed_token_ids`` - a fixed allow-list for every step.
* ``logit_bias`` - additive per-token biases.
* ``guided_choice`` - the output must be exactly one of the given alternatives (token-id lists, or strings when a
  tokenizer is attached).  The alternatives form a token trie; the allowed set of a step is the children of the node
  reached by the tokens generated so far, so the state is a pure function of the request's output and survives
  preemption and recomputation without bookkeeping.  The request stops as soon as it has produced a complete
  alternative.

* ``guided_regex`` / ``guided_json`` - the decoded output must match a regular expression (a JSON schema is first
  turned into one, for the subset in ``schema_to_regex``).  Instead of intersecting an automaton with the whole
  vocabulary, the guide tests candidates lazily: tokens are visited in descending logit order and kept when
  ``prefix + piece`` is still a partial match, until enough valid candidates are found.  Greedy decoding is exact
  (the best valid token is always found); sampling draws from the valid part of the top candidates.  Needs a
  tokenizer (token pieces come from ``decode``) and the ``regex`` package (partial matching).
Parity: the structured-outputs examples of the reference (examples/features/structured_outputs in its tree) run on
upstream's backends.
"""
from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch


class TokenTrie:
    def __init__(self, alternatives: Iterable[Sequence[int]]):
        self.root: dict = {}
        n = 0
        for alt in alternatives:
            alt = list(alt)
            if not alt:
                raise ValueError("an empty alternative cannot be generated")
            node = self.root
            for t in alt:
                node = node.setdefault(int(t), {})
            node[None] = True            # end marker
            n += 1
        if n == 0:
            raise ValueError("guided_choice needs at least one alternative")

    def _walk(self, prefix: Sequence[int]) -> Optional[dict]:
        node = self.root
        for t in prefix:
            node = node.get(int(t))
            if node is None:
                return None
        return node

    def allowed_after(self, prefix: Sequence[int]) -> list[int]:
        """Tokens that keep ``prefix`` a prefix of some alternative ([] when it is complete or off the trie)."""
        node = self._walk(prefix)
        return [] if node is None else [t for t in node if t is not None]

    def complete(self, prefix: Sequence[int]) -> bool:
        """True when ``prefix`` is an alternative and no longer one extends it - or when it left the trie."""
        node = self._walk(prefix)
        return node is None or (None in node and len(node) == 1)


def resolve_choices(choices, tokenizer) -> list[list[int]]:
    out = []
    for c in choices:
        if isinstance(c, str):
            if tokenizer is None:
                raise ValueError("string alternatives need a tokenizer; pass token-id lists instead")
            out.append(list(tokenizer.encode(c, add_special_tokens=False)))
        else:
            out.append([int(t) for t in c])
    return out


# ---------------------------------------------------------------------------------------------- regex / JSON
_JSON_WS = r"[ \n]?"
_JSON_STRING = r'"(?:[^"\\\x00-\x1f]|\\["\\/bfnrt])*"'
_JSON_NUMBER = r"-?(?:0|[1-9][0-9]*)(?:\.[0-9]+)?(?:[eE][+-]?[0-9]+)?"
_JSON_INT = r"-?(?:0|[1-9][0-9]*)"


_FORMATS = {
    "date-time": r'"\d{4}-\d{2}-\d{2}T\d{2}:\d{2}:\d{2}(?:\.\d+)?(?:Z|[+-]\d{2}:\d{2})"',
    "date": r'"\d{4}-\d{2}-\d{2}"',
    "time": r'"\d{2}:\d{2}:\d{2}(?:\.\d+)?(?:Z|[+-]\d{2}:\d{2})?"',
    "uuid": r'"[0-9a-fA-F]{8}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{12}"',
}
_STR_CHAR = r'(?:[^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'


def _any_json(depth: int) -> str:
    """Any JSON value with containers nested at most ``depth`` levels (schemas that leave a value open)."""
    scalar = f"(?:{_JSON_STRING}|{_JSON_NUMBER}|true|false|null)"
    if depth <= 0:
        return scalar
    inner = _any_json(depth - 1)
    arr = rf"\[{_JSON_WS}(?:{inner}(?:,{_JSON_WS}{inner})*)?{_JSON_WS}\]"
    member = f"{_JSON_STRING}:{_JSON_WS}{inner}"
    obj = rf"\{{{_JSON_WS}(?:{member}(?:,{_JSON_WS}{member})*)?{_JSON_WS}\}}"
    return f"(?:{scalar}|{arr}|{obj})"


# Any JSON value as a recursive group (the ``regex`` module follows ``(?&name)`` calls, also in partial matching).
_ANY_JSON_REF = "(?&jv)"
_ANY_JSON_DEFINE = (
    rf"(?(DEFINE)(?<jv>{_JSON_STRING}|{_JSON_NUMBER}|true|false|null"
    rf"|\[{_JSON_WS}(?:(?&jv)(?:,{_JSON_WS}(?&jv))*)?{_JSON_WS}\]"
    rf"|\{{{_JSON_WS}(?:{_JSON_STRING}:{_JSON_WS}(?&jv)(?:,{_JSON_WS}{_JSON_STRING}:{_JSON_WS}(?&jv))*)?{_JSON_WS}\}}))"
)


def _range_nonneg(lo: int, hi: int) -> list:
    """Alternatives (regex pieces without leading zeros) that together match exactly the integers lo..hi, 0 <= lo <= hi:
    the range is cut at the boundaries where the number of digits or a leading prefix changes."""
    if lo > hi:
        return []
    slo, shi = str(lo), str(hi)
    if len(slo) < len(shi):                       # split by digit count
        return _range_nonneg(lo, 10 ** len(slo) - 1) + _range_nonneg(10 ** len(slo), hi)
    if lo == hi:
        return [slo]
    n = len(slo)
    if n == 1:
        return [f"[{slo}-{shi}]"]
    if slo[0] == shi[0]:                          # common first digit
        return [slo[0] + (t if len(ts) == 1 else f"(?:{t})") for ts in [_range_same_len(slo[1:], shi[1:])]
                for t in ["|".join(ts)]]
    out = []
    # first digit of lo with the rest >= lo's rest, full middle digits, first digit of hi with the rest <= hi's rest
    rest_lo = _range_same_len(slo[1:], "9" * (n - 1))
    out.append(slo[0] + (rest_lo[0] if len(rest_lo) == 1 else "(?:" + "|".join(rest_lo) + ")"))
    if int(shi[0]) - int(slo[0]) > 1:
        a, b = int(slo[0]) + 1, int(shi[0]) - 1
        out.append((f"[{a}-{b}]" if a != b else str(a)) + (f"[0-9]{{{n - 1}}}" if n - 1 > 1 else "[0-9]"))
    rest_hi = _range_same_len("0" * (n - 1), shi[1:])
    out.append(shi[0] + (rest_hi[0] if len(rest_hi) == 1 else "(?:" + "|".join(rest_hi) + ")"))
    return out


def _range_same_len(slo: str, shi: str) -> list:
    """Like ``_range_nonneg`` for digit STRINGS of equal length that may start with zeros (the tail of a number)."""
    n = len(slo)
    if slo == shi:
        return [slo]
    if n == 1:
        return [f"[{slo}-{shi}]"]
    if slo == "0" * n and shi == "9" * n:
        return [f"[0-9]{{{n}}}"]
    if slo[0] == shi[0]:
        ts = _range_same_len(slo[1:], shi[1:])
        return [slo[0] + (ts[0] if len(ts) == 1 else "(?:" + "|".join(ts) + ")")]
    out = []
    ts = _range_same_len(slo[1:], "9" * (n - 1))
    out.append(slo[0] + (ts[0] if len(ts) == 1 else "(?:" + "|".join(ts) + ")"))
    if int(shi[0]) - int(slo[0]) > 1:
        a, b = int(slo[0]) + 1, int(shi[0]) - 1
        out.append((f"[{a}-{b}]" if a != b else str(a)) + (f"[0-9]{{{n - 1}}}" if n - 1 > 1 else "[0-9]"))
    ts = _range_same_len("0" * (n - 1), shi[1:])
    out.append(shi[0] + (ts[0] if len(ts) == 1 else "(?:" + "|".join(ts) + ")"))
    return out


def integer_range_regex(lo, hi) -> str:
    """Regex for the JSON integers in ``[lo, hi]``; either bound may be None (open).  Open ranges are bounded by digit
    count only where a bound exists: ``lo = 5`` gives 5..9 and every longer number."""
    alts = []
    if lo is None and hi is None:
        return _JSON_INT
    if hi is None:                                 # lo .. infinity
        if lo <= 0:
            neg = _range_nonneg(1, -lo) if lo < 0 else []
            alts += ["-" + a for a in neg] + ["0", "[1-9][0-9]*"]
        else:
            d = len(str(lo))
            alts += _range_nonneg(lo, 10 ** d - 1) + [f"[1-9][0-9]{{{d},}}"]
    elif lo is None:                               # -infinity .. hi
        if hi >= 0:
            alts += ["-[1-9][0-9]*"] + _range_nonneg(0, hi)
        else:
            d = len(str(-hi))
            alts += ["-" + a for a in _range_nonneg(-hi, 10 ** d - 1)] + [f"-[1-9][0-9]{{{d},}}"]
    else:
        if lo > hi:
            raise ValueError(f"empty integer range [{lo}, {hi}]")
        if lo < 0:
            alts += ["-" + a for a in _range_nonneg(max(1, -hi), -lo)]
        if hi >= 0:
            alts += _range_nonneg(max(lo, 0), hi)
    return "(?:" + "|".join(alts) + ")"


def _merge_all_of(parts: list) -> dict:
    """``allOf`` of object-like sub-schemas -> one schema: properties are united (a name listed twice must agree),
    ``required`` lists are united, other keywords must not conflict."""
    out: dict = {}
    for p in parts:
        for k, v in p.items():
            if k == "properties":
                props = out.setdefault("properties", {})
                for name, sub in v.items():
                    if name in props and props[name] != sub:
                        raise NotImplementedError(f"allOf: property {name!r} is constrained twice")
                    props[name] = sub
            elif k == "required":
                out["required"] = list(dict.fromkeys(out.get("required", []) + list(v)))
            elif k in out and out[k] != v:
                raise NotImplementedError(f"allOf: conflicting {k!r}")
            else:
                out[k] = v
    return out


class _RefContext:
    """The document ``$ref`` pointers resolve in, and the named group of every definition referenced so far."""

    def __init__(self, root):
        self.root = root
        self.names: dict = {}       # "#/$defs/N" -> group name
        self.defs: dict = {}        # group name -> pattern


def _schema_to_regex(schema, _root=None) -> str:
    """Regular expression for the JSON documents of a schema.

    Supported: ``type`` (one or a list of) string / integer / number / boolean / null / array / object; ``enum`` /
    ``const``; integers with ``minimum`` / ``maximum`` / ``exclusiveMinimum`` / ``exclusiveMaximum``; ``anyOf`` /
    ``oneOf`` (alternation); ``allOf`` (one part, or object parts whose properties / required lists are merged); local ``$ref`` into ``$defs`` /
    ``definitions`` (each referenced definition becomes a named group, so recursive schemas are exact); strings with ``minLength`` / ``maxLength`` /
    ``pattern`` / ``format`` (date-time, date, time, uuid); arrays with ``items`` / ``prefixItems`` / ``minItems`` /
    ``maxItems``; objects with ``properties`` in their listed order, where ``required`` (when present) says which may be
    left out - without a ``required`` list every listed property is produced; an object or schema that leaves its
    content open accepts any JSON value, nested to any depth.  Anything else raises."""
    import json
    import re

    if isinstance(schema, str):
        schema = json.loads(schema)
    ctx = _root if _root is not None else _RefContext(schema)
    root = ctx.root
    if schema is True or schema == {}:
        return _ANY_JSON_REF
    rec = lambda sub: _schema_to_regex(sub, ctx)
    if "$ref" in schema:
        ref = schema["$ref"]
        if not ref.startswith("#/"):
            raise NotImplementedError(f"only local $ref is supported: {ref!r}")
        if ref not in ctx.names:                   # one named group per referenced definition; recursion is a group call
            name = ctx.names[ref] = f"r{len(ctx.names)}"
            node = root
            for part in ref[2:].split("/"):
                node = node[part.replace("~1", "/").replace("~0", "~")]
            body = _schema_to_regex(node, ctx)
            if body == f"(?&{name})":
                raise NotImplementedError(f"$ref {ref!r} refers only to itself")
            ctx.defs[name] = body
        return f"(?&{ctx.names[ref]})"
    for key in ("anyOf", "oneOf"):
        if key in schema:
            alts = []
            for sub in schema[key]:
                alts.append(rec(sub))
            if not alts:
                raise NotImplementedError("no usable alternative")
            return "(?:" + "|".join(alts) + ")"
    if "allOf" in schema:
        parts = []
        for sub in schema["allOf"]:                # resolve references so that the parts can be merged
            while "$ref" in sub and set(sub) == {"$ref"} and sub["$ref"].startswith("#/"):
                node = root
                for part in sub["$ref"][2:].split("/"):
                    node = node[part.replace("~1", "/").replace("~0", "~")]
                sub = node
            parts.append(sub)
        rest = {k: v for k, v in schema.items() if k != "allOf"}
        return rec(parts[0] if len(parts) == 1 and not rest else _merge_all_of(parts + ([rest] if rest else [])))
    if "enum" in schema:
        return "(?:" + "|".join(re.escape(json.dumps(v)) for v in schema["enum"]) + ")"
    if "const" in schema:
        return re.escape(json.dumps(schema["const"]))
    t = schema.get("type")
    if isinstance(t, list):
        return "(?:" + "|".join(rec(dict(schema, type=one)) for one in t) + ")"
    if t is None and "properties" in schema:
        t = "object"
    if t == "string":
        if "format" in schema and schema["format"] in _FORMATS:
            return _FORMATS[schema["format"]]
        if "pattern" in schema:
            pat = schema["pattern"]
            pat = pat[1:] if pat.startswith("^") else pat
            pat = pat[:-1] if pat.endswith("$") and not pat.endswith("\\$") else pat
            return f'"(?:{pat})"'
        if "minLength" in schema or "maxLength" in schema:
            lo, hi = int(schema.get("minLength", 0)), schema.get("maxLength")
            return f'"{_STR_CHAR}{{{lo},{"" if hi is None else int(hi)}}}"'
        return _JSON_STRING
    if t == "integer":
        import math

        lo, hi = schema.get("minimum"), schema.get("maximum")
        if schema.get("exclusiveMinimum") is not None:
            lo = max(lo, schema["exclusiveMinimum"] + 1) if lo is not None else math.floor(schema["exclusiveMinimum"]) + 1
        if schema.get("exclusiveMaximum") is not None:
            hi = min(hi, schema["exclusiveMaximum"] - 1) if hi is not None else math.ceil(schema["exclusiveMaximum"]) - 1
        if lo is not None or hi is not None:
            return integer_range_regex(None if lo is None else math.ceil(lo), None if hi is None else math.floor(hi))
        return _JSON_INT
    if t == "number":
        return _JSON_NUMBER
    if t == "boolean":
        return "(?:true|false)"
    if t == "null":
        return "null"
    if t == "array":
        if "prefixItems" in schema:
            items = [rec(sub) for sub in schema["prefixItems"]]
            return rf"\[{_JSON_WS}" + f",{_JSON_WS}".join(items) + rf"{_JSON_WS}\]"
        item = rec(schema["items"]) if schema.get("items") not in (None, True) else _ANY_JSON_REF
        lo, hi = int(schema.get("minItems", 0)), schema.get("maxItems")
        more = f"(?:,{_JSON_WS}{item})"
        if hi is None:
            rest = more + ("*" if lo <= 1 else f"{{{lo - 1},}}")
        else:
            rest = more + f"{{{max(lo - 1, 0)},{max(int(hi) - 1, 0)}}}"
        body = f"{item}{rest}"
        return rf"\[{_JSON_WS}(?:{body}){'' if lo > 0 else '?'}{_JSON_WS}\]"
    if t == "object":
        props = schema.get("properties") or {}
        if not props:
            if schema.get("additionalProperties") in (None, False) and "additionalProperties" in schema:
                return r"\{" + _JSON_WS + r"\}"
            extra = schema.get("additionalProperties")
            val = rec(extra) if isinstance(extra, dict) and extra else _ANY_JSON_REF
            member = f"{_JSON_STRING}:{_JSON_WS}{val}"
            return rf"\{{{_JSON_WS}(?:{member}(?:,{_JSON_WS}{member})*)?{_JSON_WS}\}}"
        names = list(props)
        subs = [re.escape(json.dumps(k)) + ":" + _JSON_WS + rec(v) for k, v in props.items()]
        required = set(schema["required"]) if "required" in schema else set(names)
        sep = "," + _JSON_WS
        if any(n in required for n in names):
            last = max(i for i, n in enumerate(names) if n in required)
            body = ""
            for i, (n, sub) in enumerate(zip(names, subs)):
                piece = sub + sep if i < last else (sep + sub if i > last else sub)
                body += piece if n in required else f"(?:{piece})?"
        else:       # every property optional: pick which one comes first, earlier ones absent, later ones optional
            alts = []
            for i, sub in enumerate(subs):
                alts.append(sub + "".join(f"(?:{sep}{later})?" for later in subs[i + 1:]))
            body = "(?:" + "|".join(alts) + ")?"
        return r"\{" + _JSON_WS + body + _JSON_WS + r"\}"
    if t is None:
        return _ANY_JSON_REF
    raise NotImplementedError(f"JSON schema construct not supported for guided decoding: {schema!r}")


def schema_to_regex(schema) -> str:
    """Pattern (``regex`` module syntax) for the JSON documents of ``schema``; see :func:`_schema_to_regex` for the
    supported subset.  Values the schema leaves open refer to one recursive definition of "any JSON value" that is
    placed in front of the pattern, so they nest to any depth at no cost in pattern size."""
    import json

    if isinstance(schema, str):
        schema = json.loads(schema)
    ctx = _RefContext(schema)
    body = _schema_to_regex(schema, ctx)
    groups = "".join(f"(?<{name}>{sub})" for name, sub in ctx.defs.items())
    head = f"(?(DEFINE){groups})" if groups else ""
    if _ANY_JSON_REF in body or _ANY_JSON_REF in groups:
        head = _ANY_JSON_DEFINE + head
    return head + body


class RegexGuide:
    """Lazy candidate filter for one pattern (shared by the requests that use it)."""

    BATCHES = (32, 256, 2048)

    def __init__(self, pattern: str, tokenizer):
        import regex

        if tokenizer is None:
            raise ValueError("guided_regex / guided_json need a tokenizer")
        self.rx = regex.compile(pattern)
        self.tok = tokenizer
        self._piece: dict[int, str] = {}

    def piece(self, tok: int) -> str:
        p = self._piece.get(tok)
        if p is None:
            p = self.tok.decode([tok])
            self._piece[tok] = p
        return p

    def text(self, output_ids) -> str:
        return self.tok.decode(list(output_ids)) if output_ids else ""

    def is_complete(self, text: str) -> bool:
        return self.rx.fullmatch(text) is not None

    def viable(self, text: str) -> bool:
        return self.rx.fullmatch(text, partial=True) is not None

    def allowed(self, output_ids, logits_row: torch.Tensor, eos: Optional[int], want: int = 1) -> list[int]:
        """At least ``want`` valid next tokens (fewer only when the vocabulary has fewer), best logits first;
        the end-of-sequence token is valid exactly when the text so far matches the whole pattern."""
        text = self.text(output_ids)
        out: list[int] = []
        if eos is not None and self.is_complete(text):
            out.append(int(eos))
        V = logits_row.numel()
        order = None
        seen = 0
        for n in self.BATCHES + (V,):
            n = min(n, V)
            if order is None or n > len(order):
                order = torch.topk(logits_row, n).indices.tolist()
            for t in order[seen:n]:
                if t == eos:
                    continue
                p = self.piece(t)
                if p and "\ufffd" not in p and self.viable(text + p):
                    out.append(t)
            seen = n
            if len(out) >= want or n == V:
                break
        return out


def constraint_of(req) -> Optional[list[int]]:
    """Allowed token ids for the request's next step, or None when it is unconstrained."""
    p = req.params
    allowed: Optional[set] = None
    trie = getattr(p, "_trie", None)
    if trie is not None:
        nxt = trie.allowed_after(req.output_token_ids)
        if not nxt and req.eos_token_id is not None:
            nxt = [req.eos_token_id]
        allowed = set(nxt)
    if p.allowed_token_ids:
        a = set(p.allowed_token_ids)
        allowed = a if allowed is None else (allowed & a)
    return None if allowed is None else sorted(allowed)


def apply_constraints(logits: torch.Tensor, reqs) -> torch.Tensor:
    """Returns logits (a float32 copy when anything is changed) with biases added and disallowed tokens at -inf."""
    touched = False
    for i, r in enumerate(reqs):
        p = r.params
        allowed = constraint_of(r)
        guide = getattr(p, "_guide", None)
        banned = p.banned_next_tokens(r.output_token_ids) if getattr(p, "_bad_seqs", None) else []
        if allowed is None and not p.logit_bias and guide is None and not banned:
            continue
        if not touched:
            logits = logits.float().clone()
            touched = True
        if banned:                                       # bad_words: the token that would complete a banned sequence
            logits[i][torch.tensor(banned, dtype=torch.long, device=logits.device)] = float("-inf")
        if p.logit_bias:
            idx = torch.tensor(list(p.logit_bias.keys()), dtype=torch.long, device=logits.device)
            val = torch.tensor(list(p.logit_bias.values()), dtype=torch.float32, device=logits.device)
            logits[i].index_add_(0, idx, val)
        if guide is not None:
            row = logits[i].detach().float().cpu()
            if allowed is not None:                      # combine with an allow-list / choice trie
                mask = torch.full_like(row, float("-inf"))
                mask[torch.tensor(allowed, dtype=torch.long)] = 0.0
                row = row + mask
            ok = guide.allowed(r.output_token_ids, row, r.eos_token_id, want=1 if p.greedy else 16)
            if not ok and r.eos_token_id is not None:
                ok = [r.eos_token_id]                    # dead end: nothing extends the text - stop
            allowed = ok
        if allowed is not None:
            keep = torch.tensor(allowed, dtype=torch.long, device=logits.device)
            row = torch.full_like(logits[i], float("-inf"))
            row[keep] = logits[i][keep]
            logits[i] = row
    return logits
