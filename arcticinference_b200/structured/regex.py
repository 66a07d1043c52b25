"""Regular-expression guided decoding (``SamplingParams.guided_regex``): the whole
completion must match the expression.

A small regex dialect is compiled to a Thompson NFA and simulated on sets of NFA states; the
character-level machine has the same interface as the JSON-schema one
(``start / advance / advance_text / complete / exhausted``), so the same token-level matcher
(:class:`json_schema.CharMachineGrammar`) lifts it to token ids.

Supported: literals, ``.``, escapes ``\\d \\w \\s \\D \\W \\S \\n \\t`` and escaped
punctuation, classes ``[a-z0-9_]`` / ``[^...]``, groups ``( )`` and ``(?: )``, alternation
``|``, quantifiers ``? * + {m} {m,} {m,n}`` (greedy or lazy makes no difference to a
full match). ``^`` at the start and ``$`` at the end are accepted and ignored. Back
references and look-around are not regular and raise ``ValueError``.
"""

from __future__ import annotations

from typing import Optional

_MAX_REPEAT = 256
_WORD = set("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789_")
_SPACE = set(" \t\n\r\f\v")
_DIGIT = set("0123456789")


class _Pred:
    """A set of characters, possibly negated ('.' is everything but a line feed)."""
    __slots__ = ("chars", "negated")

    def __init__(self, chars, negated=False):
        self.chars, self.negated = frozenset(chars), negated

    def __call__(self, ch: str) -> bool:
        return (ch in self.chars) != self.negated


def _escape_pred(c: str) -> _Pred:
    table = {"d": (_DIGIT, False), "D": (_DIGIT, True), "w": (_WORD, False), "W": (_WORD, True),
             "s": (_SPACE, False), "S": (_SPACE, True)}
    if c in table:
        return _Pred(*table[c])
    if c in "nrtfv":
        return _Pred({"n": "\n", "r": "\r", "t": "\t", "f": "\f", "v": "\v"}[c])
    if c.isdigit() or c in "bBAZ":
        raise ValueError("unsupported escape \\%s" % c)
    return _Pred(c)


# --------------------------------------------------------------------------- parser -> AST
# AST: ("char", pred) | ("cat", [nodes]) | ("alt", [nodes]) | ("rep", node, lo, hi|None)
class _Parser:
    def __init__(self, text: str):
        self.t, self.i = text, 0

    def peek(self) -> Optional[str]:
        return self.t[self.i] if self.i < len(self.t) else None

    def take(self) -> str:
        c = self.t[self.i]
        self.i += 1
        return c

    def parse(self):
        if self.peek() == "^":
            self.take()
        node = self.alternation()
        if self.i != len(self.t):
            raise ValueError("unbalanced ')' at %d" % self.i)
        return node

    def alternation(self):
        options = [self.concatenation()]
        while self.peek() == "|":
            self.take()
            options.append(self.concatenation())
        return options[0] if len(options) == 1 else ("alt", options)

    def concatenation(self):
        items = []
        while self.peek() is not None and self.peek() not in "|)":
            if self.peek() == "$" and self.i == len(self.t) - 1:
                self.take()
                break
            items.append(self.quantified())
        return ("cat", items)

    def quantified(self):
        atom = self.atom()
        while self.peek() is not None and self.peek() in "?*+{":
            c = self.peek()
            if c == "{":
                j = self.t.find("}", self.i)
                body = self.t[self.i + 1:j] if j > 0 else ""
                parts = body.split(",")
                if j < 0 or not all(p.strip().isdigit() or p.strip() == "" for p in parts) or \
                        len(parts) > 2 or not parts[0].strip().isdigit():
                    raise ValueError("bad repetition at %d" % self.i)
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                self.i = j + 1
            else:
                self.take()
                lo, hi = {"?": (0, 1), "*": (0, None), "+": (1, None)}[c]
            if hi is not None and (hi < lo or hi > _MAX_REPEAT) or lo > _MAX_REPEAT:
                raise ValueError("repetition bounds out of range")
            if self.peek() == "?":
                self.take()        # a lazy quantifier matches the same full strings
            atom = ("rep", atom, lo, hi)
        return atom

    def atom(self):
        c = self.take()
        if c == "(":
            if self.t.startswith("?:", self.i):
                self.i += 2
            elif self.peek() == "?":
                raise ValueError("look-around and named groups are not supported")
            node = self.alternation()
            if self.peek() != ")":
                raise ValueError("missing ')'")
            self.take()
            return node
        if c == "[":
            return ("char", self.char_class())
        if c == ".":
            return ("char", _Pred("\n", True))
        if c == "\\":
            if self.peek() is None:
                raise ValueError("dangling backslash")
            return ("char", _escape_pred(self.take()))
        if c in "*+?{":
            raise ValueError("nothing to repeat at %d" % (self.i - 1))
        return ("char", _Pred(c))

    def char_class(self) -> _Pred:
        negated = self.peek() == "^"
        if negated:
            self.take()
        chars, extra = set(), []
        first = True
        while True:
            if self.peek() is None:
                raise ValueError("missing ']'")
            c = self.take()
            if c == "]" and not first:
                break
            first = False
            if c == "\\":
                p = _escape_pred(self.take())
                if p.negated:
                    extra.append(p)
                else:
                    chars |= p.chars
                continue
            if self.peek() == "-" and self.i + 1 < len(self.t) and self.t[self.i + 1] != "]":
                self.take()
                hi = self.take()
                if hi == "\\":
                    hi = self.take()
                if ord(hi) < ord(c):
                    raise ValueError("bad range %s-%s" % (c, hi))
                chars |= {chr(x) for x in range(ord(c), ord(hi) + 1)}
            else:
                chars.add(c)
        if extra:
            raise ValueError("negated escapes inside a class are not supported")
        return _Pred(chars, negated)


# ----------------------------------------------------------------------------- NFA
class CompiledRegex:
    """Thompson NFA. ``trans[s]`` is a list of (predicate, target); ``eps[s]`` a list of
    targets; one accepting state."""

    def __init__(self, pattern: str):
        self.pattern = pattern
        self.trans: list = []
        self.eps: list = []
        ast = _Parser(pattern).parse()
        s0 = self._new()
        self.accept = self._build(ast, s0)
        self._closure_cache: dict = {}
        self._start = self._close({s0})
        self.allowed_cache: dict = {}

    def _new(self) -> int:
        self.trans.append([])
        self.eps.append([])
        return len(self.trans) - 1

    def _build(self, node, start: int) -> int:
        """Wire ``node`` from ``start``; returns its end state."""
        kind = node[0]
        if kind == "char":
            end = self._new()
            self.trans[start].append((node[1], end))
            return end
        if kind == "cat":
            cur = start
            for item in node[1]:
                cur = self._build(item, cur)
            return cur
        if kind == "alt":
            end = self._new()
            for opt in node[1]:
                s = self._new()
                self.eps[start].append(s)
                self.eps[self._build(opt, s)].append(end)
            return end
        if kind == "rep":
            _, sub, lo, hi = node
            cur = start
            for _ in range(lo):
                cur = self._build(sub, cur)
            if hi is None:
                loop = self._new()
                self.eps[cur].append(loop)
                self.eps[self._build(sub, loop)].append(loop)
                return loop
            end = self._new()
            self.eps[cur].append(end)
            for _ in range(hi - lo):
                cur = self._build(sub, cur)
                self.eps[cur].append(end)
            return end
        raise ValueError("bad node %r" % (node,))

    def _close(self, states) -> frozenset:
        out, todo = set(states), list(states)
        while todo:
            for t in self.eps[todo.pop()]:
                if t not in out:
                    out.add(t)
                    todo.append(t)
        return frozenset(out)

    # machine interface
    def start(self) -> frozenset:
        return self._start

    def advance(self, state: frozenset, ch: str) -> Optional[frozenset]:
        nxt = {t for s in state for pred, t in self.trans[s] if pred(ch)}
        return self._close(nxt) if nxt else None

    def advance_text(self, state: frozenset, text: str) -> Optional[frozenset]:
        for ch in text:
            state = self.advance(state, ch)
            if state is None:
                return None
        return state

    def complete(self, state: frozenset) -> bool:
        return self.accept in state

    def exhausted(self, state: frozenset) -> bool:
        return self.accept in state and not any(self.trans[s] for s in state)

    def validate(self, text: str) -> bool:
        st = self.advance_text(self.start(), text)
        return st is not None and self.complete(st)


_COMPILED: dict = {}


def compile_regex(pattern: str) -> CompiledRegex:
    c = _COMPILED.get(pattern)
    if c is None:
        if len(_COMPILED) > 256:
            _COMPILED.clear()
        c = _COMPILED[pattern] = CompiledRegex(pattern)
    return c
