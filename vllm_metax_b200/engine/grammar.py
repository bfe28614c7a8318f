"""``guided_grammar``: a context-free grammar in GBNF / EBNF notation turned into ONE recursive pattern.

The ``regex`` module follows named-group calls ``(?&rule)`` - also in partial matching, which is what the guide of
``guided_regex`` uses to test a candidate token against the text so far - so a grammar needs no automaton of its own:
every rule becomes a named group inside a ``(?(DEFINE)...)`` block, a rule reference becomes a call of its group, and
the pattern's body calls ``root``.  The guide, its candidate batching and its caches are then the ones of
``guided_regex`` (engine/structured.py).

Notation (the subset upstream's grammar backend documents for ``guided_grammar``):

    root   ::= "SELECT " column " FROM " table (" WHERE " cond)?
    column ::= "name" | "age"            # alternatives
    table  ::= [a-z_]+                   # character classes, negated with ^
    cond   ::= column " = " [0-9]{1,3}   # * + ? {m} {m,} {m,n} repeat the item before them
    any    ::= .                         # any character

String literals take ``\\n \\r \\t \\" \\\\ \\xHH \\uHHHH``; ``#`` starts a comment; a rule may continue on the next
lines; rule names may contain ``-``.  Left recursion (``expr ::= expr "+" term``) cannot be followed by a backtracking
matcher and is refused with the cycle named; write it as repetition (``expr ::= term ("+" term)*``).

Parity: upstream's structured-output backends accept EBNF grammars (``SamplingParams.structured_outputs.grammar``);
the reference inherits them.
"""
from __future__ import annotations

import re

_RULE_HEAD = re.compile(r"^[ \t]*([A-Za-z_][A-Za-z0-9_-]*)[ \t]*::=", re.M)
_ESC = {"n": "\n", "r": "\r", "t": "\t", '"': '"', "\\": "\\", "'": "'", "[": "[", "]": "]", "-": "-", "^": "^"}


def _strip_comments(text: str) -> str:
    out, i, n = [], 0, len(text)
    quote, in_class = None, False
    while i < n:
        c = text[i]
        if c == "\\" and (quote or in_class) and i + 1 < n:
            out.append(text[i:i + 2])
            i += 2
            continue
        if quote:
            quote = None if c == quote else quote
        elif in_class:
            in_class = c != "]"
        elif c in "\"'":
            quote = c
        elif c == "[":
            in_class = True
        elif c == "#":
            while i < n and text[i] != "\n":
                i += 1
            continue
        out.append(c)
        i += 1
    return "".join(out)


class _RuleParser:
    """Recursive descent over one rule body; produces the pattern and the rules that can start a match of it."""

    def __init__(self, name: str, body: str, group_of, nullable_rules=frozenset()):
        self.name, self.s, self.i, self.group_of = name, body, 0, group_of
        self.nullable_rules = nullable_rules
        self.refs: set = set()

    def fail(self, msg: str):
        raise ValueError(f"grammar rule {self.name!r}, offset {self.i}: {msg}")

    def ws(self):
        while self.i < len(self.s) and self.s[self.i] in " \t\r\n":
            self.i += 1

    def escape(self) -> str:
        """After a backslash: the character it stands for."""
        c = self.s[self.i]
        self.i += 1
        if c in "xu":
            k = 2 if c == "x" else 4
            h = self.s[self.i:self.i + k]
            if len(h) != k or not all(x in "0123456789abcdefABCDEF" for x in h):
                self.fail(f"\\{c} needs {k} hex digits")
            self.i += k
            return chr(int(h, 16))
        if c not in _ESC:
            self.fail(f"unknown escape \\{c}")
        return _ESC[c]

    def alternatives(self, closer: str):
        """-> (pattern, nullable, leftmost rule references)"""
        alts, nullable, left = [], False, set()
        while True:
            p, nl, lf = self.sequence(closer)
            alts.append(p)
            nullable |= nl
            left |= lf
            self.ws()
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                continue
            break
        return ("(?:" + "|".join(alts) + ")" if len(alts) > 1 else alts[0]), nullable, left

    def sequence(self, closer: str):
        parts, nullable, left = [], True, set()
        while True:
            self.ws()
            if self.i >= len(self.s) or self.s[self.i] in "|" + closer:
                break
            p, nl, lf = self.item()
            if nullable:                 # everything before this item can be empty: it can start the match
                left |= lf
            nullable &= nl
            parts.append(p)
        return "".join(parts), nullable, left

    def item(self):
        c = self.s[self.i]
        if c in "\"'":
            self.i += 1
            chars = []
            while True:
                if self.i >= len(self.s):
                    self.fail("unterminated string")
                d = self.s[self.i]
                self.i += 1
                if d == c:
                    break
                chars.append(self.escape() if d == "\\" else d)
            text = "".join(chars)
            p, nl, lf = (re.escape(text) if len(text) <= 1 else "(?:" + re.escape(text) + ")"), not text, set()
        elif c == "[":
            self.i += 1
            out = ["["]
            if self.i < len(self.s) and self.s[self.i] == "^":
                out.append("^")
                self.i += 1
            while True:
                if self.i >= len(self.s):
                    self.fail("unterminated character class")
                d = self.s[self.i]
                self.i += 1
                if d == "]":
                    break
                if d == "-" and len(out) > 1 and self.i < len(self.s) and self.s[self.i] != "]":
                    out.append("-")
                    continue
                ch = self.escape() if d == "\\" else d
                out.append("\\" + ch if ch in "\\]^-[&~|" else ("\\n" if ch == "\n" else ch))
            if out in (["["], ["[", "^"]):
                self.fail("empty character class")
            p, nl, lf = "".join(out) + "]", False, set()
        elif c == "(":
            self.i += 1
            p, nl, lf = self.alternatives(")")
            self.ws()
            if self.i >= len(self.s) or self.s[self.i] != ")":
                self.fail("missing )")
            self.i += 1
            p = p if p.startswith("(?:") and p.endswith(")") and _balanced(p) else f"(?:{p})"
        elif c == ".":
            self.i += 1
            p, nl, lf = r"(?s:.)", False, set()
        elif c.isalpha() or c == "_":
            j = self.i
            while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "_-"):
                j += 1
            ref = self.s[self.i:j]
            self.i = j
            self.refs.add(ref)
            p, nl, lf = f"(?&{self.group_of(ref)})", ref in self.nullable_rules, {ref}
        else:
            self.fail(f"unexpected {c!r}")
        # repetition
        while self.i < len(self.s) and self.s[self.i] in "*+?{":
            q = self.s[self.i]
            if q == "{":
                m = re.match(r"\{(\d+)(?:(,)(\d*))?\}", self.s[self.i:])
                if not m:
                    self.fail("malformed {m,n}")
                lo = int(m.group(1))
                hi = lo if not m.group(2) else (int(m.group(3)) if m.group(3) else None)
                if hi is not None and hi < lo:
                    self.fail("{m,n} with n < m")
                self.i += m.end()
                p += f"{{{lo}}}" if hi == lo else (f"{{{lo},}}" if hi is None else f"{{{lo},{hi}}}")
                nl = nl or lo == 0
            else:
                self.i += 1
                p += q
                nl = nl or q in "*?"
            p = f"(?:{p})"
        return p, nl, lf


def _balanced(p: str) -> bool:
    """True when the outer ``(?:`` of ``p`` closes at its last character (so no second wrapping is needed)."""
    depth, i, in_class = 0, 0, False
    while i < len(p):
        c = p[i]
        if c == "\\":
            i += 2
            continue
        if in_class:
            in_class = c != "]"
        elif c == "[":
            in_class = True
        elif c == "(":
            depth += 1
        elif c == ")":
            depth -= 1
            if depth == 0 and i != len(p) - 1:
                return False
        i += 1
    return depth == 0


def grammar_to_regex(grammar: str, root: str = "root") -> str:
    """Pattern (``regex`` module syntax) that matches exactly the strings of ``grammar`` derived from ``root``."""
    text = _strip_comments(grammar)
    heads = list(_RULE_HEAD.finditer(text))
    if not heads:
        raise ValueError("the grammar has no rule (name ::= ...)")
    if text[:heads[0].start()].strip():
        raise ValueError(f"text before the first rule: {text[:heads[0].start()].strip()[:40]!r}")
    bodies: dict = {}
    for k, h in enumerate(heads):
        name = h.group(1)
        if name in bodies:
            raise ValueError(f"rule {name!r} is defined twice")
        bodies[name] = text[h.end(): heads[k + 1].start() if k + 1 < len(heads) else len(text)]
    if root not in bodies:
        raise ValueError(f"the grammar has no {root!r} rule")
    names = {name: "g_" + re.sub(r"[^A-Za-z0-9_]", "_", name) + (f"_{i}" if "-" in name else "") for i, name in enumerate(bodies)}

    def group_of(ref: str) -> str:
        if ref not in names:
            raise ValueError(f"rule {ref!r} is used but not defined")
        return names[ref]

    # Parse until the set of rules that can match the empty string stops growing (a reference to such a rule does
    # not consume, so what follows it can still start the match).
    can_be_empty: set = set()
    while True:
        patterns, nullable, leftmost = {}, {}, {}
        for name, body in bodies.items():
            rp = _RuleParser(name, body, group_of, frozenset(can_be_empty))
            p, nl, lf = rp.alternatives("")
            rp.ws()
            if rp.i != len(rp.s):
                rp.fail(f"unexpected {rp.s[rp.i]!r}")
            patterns[name], nullable[name], leftmost[name] = p, nl, lf
        grown = {n for n, nl in nullable.items() if nl}
        if grown == can_be_empty:
            break
        can_be_empty = grown
    # Left recursion: a rule that can call itself before consuming anything.
    reach = {n: set(lf) for n, lf in leftmost.items()}
    changed = True
    while changed:
        changed = False
        for n in reach:
            more = set().union(*(reach[m] for m in reach[n])) - reach[n] if reach[n] else set()
            if more:
                reach[n] |= more
                changed = True
    loops = sorted(n for n in reach if n in reach[n])
    if loops:
        raise NotImplementedError(f"left-recursive grammar rule(s) {loops}: rewrite as repetition, e.g. "
                                  "expr ::= term (op term)*")
    groups = "".join(f"(?<{names[n]}>{p})" for n, p in patterns.items())
    return f"(?(DEFINE){groups})(?&{names[root]})"
