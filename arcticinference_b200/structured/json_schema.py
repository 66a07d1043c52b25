"""JSON-schema guided decoding: a character-level matcher compiled from a schema, lifted to
token ids through the tokenizer's vocabulary.

The reference gets guided JSON from vLLM's grammar back end and evaluates it with its
JSON-mode benchmark (tests/benchmarks/json_mode/task_description.py:6-33: flat and nested
pydantic models with string / number / list fields). This module covers that subset of JSON
Schema natively: ``object`` (properties in declaration order; with a ``required`` list the
other properties are optional), ``array`` (``items``, ``minItems``, ``maxItems``),
``string`` (``maxLength``, ``enum``, anchored ``pattern``), ``integer``, ``number``, ``boolean``, ``null``,
``enum`` / ``const`` of any JSON literals, ``anyOf`` / ``oneOf`` / lists of types, and
``$ref`` into ``$defs`` / ``definitions``. Output is compact JSON (no white space).

The matcher is a stack machine. One reading of the text so far is a tuple of frames; a
state is the set of readings that are still possible (alternatives fork it), hashable, so
the set of allowed tokens is computed once per distinct state and shared by every request
that uses the same compiled schema.
"""

from __future__ import annotations

import json
from typing import Optional, Sequence

import numpy as np

from . import Grammar

_MAX_CACHED_STATES = 1024
_DIGITS = "0123456789"
_HEX = "0123456789abcdefABCDEF"
_ESCAPES = '"\\/bfnrt'


# ---------------------------------------------------------------------------- compilation
class _Node:
    """kind: lit | str | re | int | num | trie | seq | arr | alt (``re``: a string whose
    characters match a regular expression; its machine sits in the ``trie`` slot)"""
    __slots__ = ("kind", "text", "max_len", "trie", "children", "item", "min_items", "max_items")

    def __init__(self, kind, **kw):
        self.kind = kind
        self.text = kw.get("text")
        self.max_len = kw.get("max_len")
        self.trie = kw.get("trie")
        self.children = kw.get("children")
        self.item = kw.get("item")
        self.min_items = kw.get("min_items", 0)
        self.max_items = kw.get("max_items")


def _make_trie(words: Sequence[str]):
    """Nested dicts; the key None marks the end of a word."""
    root: dict = {}
    for w in words:
        node = root
        for ch in w:
            node = node.setdefault(ch, {})
        node[None] = True
    return root


class CompiledSchema:
    def __init__(self, schema):
        if isinstance(schema, str):
            schema = json.loads(schema)
        self.schema = schema
        self.nodes: list[_Node] = []
        self._defs = {}
        for key in ("$defs", "definitions"):
            self._defs.update(schema.get(key, {}) if isinstance(schema, dict) else {})
        self.root = self._compile(schema, 0)
        self.allowed_cache: dict = {}     # (vocabulary id, state) -> list of token ids

    def _alt(self, options: list) -> int:
        if len(options) == 1:
            return options[0]
        return self._add(_Node("alt", children=options))

    def _add(self, node: _Node) -> int:
        self.nodes.append(node)
        return len(self.nodes) - 1

    def _compile(self, sch, depth: int) -> int:
        if depth > 32:
            raise ValueError("schema nests too deeply (recursive $ref?)")
        if sch is True or sch == {}:
            raise ValueError("unconstrained sub-schemas are not supported")
        if "$ref" in sch:
            name = sch["$ref"].split("/")[-1]
            if name not in self._defs:
                raise ValueError("unresolved $ref %r" % sch["$ref"])
            return self._compile(self._defs[name], depth + 1)
        if "const" in sch:
            return self._add(_Node("lit", text=json.dumps(sch["const"], separators=(",", ":"))))
        if "enum" in sch:
            words = [json.dumps(v, separators=(",", ":")) for v in sch["enum"]]
            return self._add(_Node("trie", trie=_make_trie(words)))
        for key in ("anyOf", "oneOf"):
            if key in sch:
                return self._alt([self._compile(o, depth + 1) for o in sch[key]])
        t = sch.get("type")
        if isinstance(t, list):
            rest = {k: v for k, v in sch.items() if k != "type"}
            return self._alt([self._compile(dict(rest, type=one), depth + 1) for one in t])
        if t == "string":
            if "pattern" in sch:
                # the pattern constrains the raw characters between the quotes; characters
                # that would need escaping in JSON are never allowed there
                from .regex import compile_regex
                pat = sch["pattern"]
                if not (pat.startswith("^") and pat.endswith("$")):
                    raise ValueError("string patterns must be anchored (^...$): an unanchored "
                                     "pattern constrains nothing a grammar can enforce")
                return self._add(_Node("re", text=pat, trie=compile_regex(pat),
                                       max_len=sch.get("maxLength")))
            return self._add(_Node("str", max_len=sch.get("maxLength")))
        if t == "integer":
            return self._add(_Node("int"))
        if t == "number":
            return self._add(_Node("num"))
        if t == "boolean":
            return self._add(_Node("trie", trie=_make_trie(["true", "false"])))
        if t == "null":
            return self._add(_Node("lit", text="null"))
        if t == "array":
            item = self._compile(sch.get("items", {}), depth + 1)
            return self._add(_Node("arr", item=item, min_items=int(sch.get("minItems", 0)),
                                   max_items=sch.get("maxItems")))
        if t == "object" or "properties" in sch:
            props = list(sch.get("properties", {}).items())
            if not props:
                return self._add(_Node("lit", text="{}"))
            # Properties come in declaration order. With a "required" list the others may be
            # left out: tail(i, emitted) is what may follow once the first i properties have
            # been dealt with, ``emitted`` telling whether a separator is due.
            required = set(sch["required"]) if "required" in sch else {k for k, _ in props}
            values = [self._compile(sub, depth + 1) for _, sub in props]
            memo: dict = {}

            def tail(i: int, emitted: bool) -> int:
                key = (i, emitted)
                if key in memo:
                    return memo[key]
                if i == len(props):
                    nid = self._add(_Node("lit", text="}"))
                else:
                    name = props[i][0]
                    lead = self._add(_Node("lit", text=("," if emitted else "") +
                                           json.dumps(name) + ":"))
                    taken = self._add(_Node("seq", children=[lead, values[i], tail(i + 1, True)]))
                    nid = taken if name in required else self._alt([taken, tail(i + 1, emitted)])
                memo[key] = nid
                return nid

            return self._add(_Node("seq", children=[self._add(_Node("lit", text="{")),
                                                    tail(0, False)]))
        raise ValueError("unsupported schema: %r" % (sch,))

    # ------------------------------------------------------------------------ machine
    # frames: (node id, a, b) -- the meaning of a, b depends on the node kind
    def start(self) -> frozenset:
        return frozenset([(self._enter(self.root),)])

    def _enter(self, nid: int) -> tuple:
        n = self.nodes[nid]
        if n.kind == "trie":
            return (nid, (), 0)            # a = path of characters into the trie
        if n.kind == "re":
            return (nid, None, 0)          # a = set of NFA states (None before the quote)
        return (nid, 0, 0)

    def _trie_at(self, n: _Node, path: tuple) -> dict:
        node = n.trie
        for ch in path:
            node = node[ch]
        return node

    def _accepting(self, frame) -> bool:
        """May this frame end here (without consuming anything more)?"""
        nid, a, b = frame
        n = self.nodes[nid]
        k = n.kind
        if k == "lit":
            return a == len(n.text)
        if k == "str":
            return a == 9
        if k == "re":
            return a == 9
        if k == "int":
            return a in (2, 3)
        if k == "num":
            return a in (2, 3, 5, 8)
        if k == "trie":
            return None in self._trie_at(n, a)
        if k == "seq":
            return a == len(n.children)
        if k == "arr":
            return a == 9
        return False      # alt: no JSON value is empty

    def _consume_leaf(self, frame, ch: str):
        """One character into a frame of a leaf kind (lit, trie, str, int, num): the frame
        that replaces it, as a one-element tuple, or None if ``ch`` does not fit."""
        nid, a, b = frame
        n = self.nodes[nid]
        k = n.kind
        if k == "lit":
            if a < len(n.text) and n.text[a] == ch:
                return ((nid, a + 1, 0),)
            return None
        if k == "trie":
            node = self._trie_at(n, a)
            if ch in node:
                return ((nid, a + (ch,), 0),)
            return None
        if k == "re":
            rx = n.trie
            if a is None:
                return ((nid, rx.start(), 0),) if ch == '"' else None
            if a == 9:
                return None
            if ch == '"':
                return ((nid, 9, b),) if rx.complete(a) else None
            if ch == "\\" or ord(ch) < 0x20 or (n.max_len is not None and b >= n.max_len):
                return None
            nxt = rx.advance(a, ch)
            if nxt is None:
                return None
            return ((nid, nxt, b + 1 if n.max_len is not None else 0),)
        if k == "str":
            # a: 0 before the opening quote, 1 inside, 2 after a backslash, 3..6 the four hex
            # digits of \uXXXX, 9 closed; b counts characters when maxLength is set
            if a == 0:
                return ((nid, 1, 0),) if ch == '"' else None
            if a == 1:
                if ch == '"':
                    return ((nid, 9, b),)
                if ch == "\\":
                    if n.max_len is not None and b >= n.max_len:
                        return None          # no room for the escaped character
                    return ((nid, 2, b),)
                if ord(ch) < 0x20:
                    return None
                if n.max_len is not None:
                    if b >= n.max_len:
                        return None
                    return ((nid, 1, b + 1),)
                return ((nid, 1, 0),)
            if a == 2:
                nb = b + 1 if n.max_len is not None else 0
                if ch in _ESCAPES:
                    return ((nid, 1, nb),)
                if ch == "u":
                    return ((nid, 3, nb),)
                return None
            if 3 <= a <= 6:
                if ch in _HEX:
                    return ((nid, 1 if a == 6 else a + 1, b),)
                return None
            return None
        if k in ("int", "num"):
            # 0 start, 1 after '-', 2 after a lone 0, 3 in the integer digits,
            # 4 after '.', 5 fraction digits, 6 after e/E, 7 after the exponent sign, 8 exponent
            if a == 0:
                if ch == "-":
                    return ((nid, 1, 0),)
                if ch == "0":
                    return ((nid, 2, 0),)
                return ((nid, 3, 0),) if ch in "123456789" else None
            if a == 1:
                if ch == "0":
                    return ((nid, 2, 0),)
                return ((nid, 3, 0),) if ch in "123456789" else None
            if a == 3 and ch in _DIGITS:
                return ((nid, 3, b + 1),) if b < 30 else None
            if k == "int":
                return None
            if a in (2, 3) and ch == ".":
                return ((nid, 4, 0),)
            if a in (2, 3, 5) and ch in "eE":
                return ((nid, 6, 0),)
            if a in (4, 5) and ch in _DIGITS:
                return ((nid, 5, b + 1),) if b < 30 else None
            if a == 6 and ch in "+-":
                return ((nid, 7, 0),)
            if a in (6, 7, 8) and ch in _DIGITS:
                # at most two exponent digits: every accepted number is a finite double
                return ((nid, 8, b + 1),) if b < 2 else None
            return None
        return None

    def _consume(self, frame, ch: str) -> list:
        """One character into the top frame: every way it can be taken, each as the tuple of
        frames that replaces the frame (itself, possibly with children pushed above it).
        Empty when ``ch`` does not fit. seq and arr push their child and let it consume; alt
        forks into its options."""
        nid, a, b = frame
        n = self.nodes[nid]
        k = n.kind
        if k == "alt":
            out = []
            for c in n.children:
                out.extend(self._consume(self._enter(c), ch))
            return out
        if k == "seq":
            if a >= len(n.children):
                return []
            return [((nid, a + 1, 0),) + got
                    for got in self._consume(self._enter(n.children[a]), ch)]
        if k == "arr":
            # a: 0 before '[', 1 right after '[', 2 after an item, 3 after ',', 9 closed;
            # b items so far
            if a == 0:
                return [((nid, 1, 0),)] if ch == "[" else []
            if a == 1 or a == 3:
                if a == 1 and ch == "]":
                    return [((nid, 9, b),)] if b >= n.min_items else []
                if n.max_items is not None and b >= n.max_items:
                    return []
                return [((nid, 2, b + 1),) + got
                        for got in self._consume(self._enter(n.item), ch)]
            if a == 2:
                if ch == ",":
                    if n.max_items is not None and b >= n.max_items:
                        return []
                    return [((nid, 3, b),)]
                if ch == "]":
                    return [((nid, 9, b),)] if b >= n.min_items else []
            return []
        got = self._consume_leaf(frame, ch)
        return [] if got is None else [got]

    def _advance_stack(self, stack: tuple, ch: str) -> list:
        """Stacks reachable from one stack by ``ch``. Finished frames on top are popped when
        they cannot take the character themselves (numbers end by look-ahead)."""
        frames = list(stack)
        while frames:
            alts = self._consume(frames[-1], ch)
            if alts:
                out = []
                for got in alts:
                    new = frames[:-1] + list(got)
                    # drop frames that can take nothing more (closed literals, strings, ...)
                    while new and self._closed(new[-1]):
                        new.pop()
                    out.append(tuple(new))
                return out
            if not self._accepting(frames[-1]):
                return []
            frames.pop()
        return []

    def advance(self, state: frozenset, ch: str) -> Optional[frozenset]:
        """State (a set of stacks, one per way of reading the text so far) after ``ch``, or
        None when no reading survives."""
        out = set()
        for stack in state:
            out.update(self._advance_stack(stack, ch))
        return frozenset(out) if out else None

    def _closed(self, frame) -> bool:
        nid, a, b = frame
        n = self.nodes[nid]
        k = n.kind
        if k == "lit":
            return a == len(n.text)
        if k in ("str", "arr", "re"):
            return a == 9
        if k == "seq":
            return a == len(n.children)
        if k == "trie":
            node = self._trie_at(n, a)
            return None in node and len(node) == 1
        return False

    def advance_text(self, state: frozenset, text: str) -> Optional[frozenset]:
        for ch in text:
            state = self.advance(state, ch)
            if state is None:
                return None
        return state

    def complete(self, state: frozenset) -> bool:
        """True when the text so far is a whole document under some reading."""
        return any(all(self._accepting(f) for f in stack) for stack in state)

    def exhausted(self, state: frozenset) -> bool:
        """True when the document is whole and nothing can follow it."""
        return all(len(stack) == 0 for stack in state)

    def validate(self, text: str) -> bool:
        st = self.advance_text(self.start(), text)
        return st is not None and self.complete(st)


# ------------------------------------------------------------------------- vocabulary
class Vocabulary:
    """Token id -> text, with the tokens grouped by first character so that a state only
    tries tokens whose first character it can take."""

    _next_id = 0

    def __init__(self, strings: Sequence[Optional[str]]):
        self.strings = list(strings)
        self.by_first: dict = {}
        for tid, s in enumerate(self.strings):
            if s:
                self.by_first.setdefault(s[0], []).append(tid)
        Vocabulary._next_id += 1
        self.uid = Vocabulary._next_id

    @classmethod
    def from_tokenizer(cls, tokenizer, vocab_size: int) -> "Vocabulary":
        cached = getattr(tokenizer, "_ab200_vocabulary", None)
        if cached is not None and len(cached.strings) == vocab_size:
            return cached
        special = {getattr(tokenizer, a, None) for a in ("bos_token_id", "eos_token_id",
                                                           "pad_token_id")}
        strings: list = []
        for tid in range(vocab_size):
            if tid in special:
                strings.append(None)
                continue
            try:
                s = tokenizer.decode([tid], skip_special_tokens=False)
            except Exception:  # noqa: BLE001 - ids without a token
                s = None
            # a token that is only part of a multi-byte character decodes to U+FFFD
            strings.append(s if s and "�" not in s else None)
        v = cls(strings)
        try:
            tokenizer._ab200_vocabulary = v
        except Exception:  # noqa: BLE001 - tokenizers that refuse new attributes
            pass
        return v


class CharMachineGrammar(Grammar):
    """Token-level matcher for one sequence over a character-level machine (a compiled JSON
    schema or regular expression: ``start / advance / advance_text / complete / exhausted``
    and an ``allowed_cache`` dict). ``eos_token_id`` is allowed once the text is a whole
    document; a document that cannot be extended finishes by itself."""

    def __init__(self, compiled, vocab: Vocabulary, eos_token_id: Optional[int] = None):
        self.c, self.v, self.eos = compiled, vocab, eos_token_id
        self._hist = [compiled.start()]
        self._ended = False

    @property
    def state(self) -> tuple:
        return self._hist[-1]

    @property
    def finished(self) -> bool:
        return self._ended or self.c.exhausted(self.state)

    def allowed(self):
        """Allowed token ids as an int64 array (shared with the cache: do not modify)."""
        if self.finished:
            return np.asarray([self.eos] if self.eos is not None else [], dtype=np.int64)
        st = self.state
        key = (self.v.uid, st)
        cache = self.c.allowed_cache
        toks = cache.get(key)
        if toks is None:
            ids = []
            for first, tids in self.v.by_first.items():
                if self.c.advance(st, first) is None:
                    continue
                for tid in tids:
                    s = self.v.strings[tid]
                    if len(s) == 1 or self.c.advance_text(st, s) is not None:
                        ids.append(tid)
            toks = np.asarray(sorted(ids), dtype=np.int64)
            if len(cache) >= _MAX_CACHED_STATES:
                cache.clear()       # bounded: a state's list can be as long as the vocabulary
            cache[key] = toks
        if self.eos is not None and self.c.complete(st):
            return np.append(toks, self.eos)
        return toks

    def accept(self, token: int) -> bool:
        if self.finished:
            return False
        st = self.state
        if self.eos is not None and token == self.eos:
            if not self.c.complete(st):
                return False
            self._hist.append(st)
            self._ended = True
            return True
        s = self.v.strings[token] if 0 <= token < len(self.v.strings) else None
        if not s:
            return False
        nxt = self.c.advance_text(st, s)
        if nxt is None:
            return False
        self._hist.append(nxt)
        return True

    def rollback(self, n: int) -> None:
        if n <= 0:
            return
        if n >= len(self._hist):
            raise ValueError("cannot roll back %d of %d tokens" % (n, len(self._hist) - 1))
        del self._hist[-n:]
        self._ended = False


JsonSchemaGrammar = CharMachineGrammar


_COMPILED: dict = {}


def compile_schema(schema) -> CompiledSchema:
    """Compiled form of a schema, shared by all requests that use the same one."""
    key = schema if isinstance(schema, str) else json.dumps(schema, sort_keys=False)
    c = _COMPILED.get(key)
    if c is None:
        if len(_COMPILED) > 256:
            _COMPILED.clear()
        c = _COMPILED[key] = CompiledSchema(schema)
    return c
