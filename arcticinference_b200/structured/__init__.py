"""Structured (grammar-constrained) outputs that cooperate with speculative decoding.

A grammar is a deterministic matcher over token ids: it says which tokens may come next,
advances over accepted tokens, and can take back the most recent ones. The take-back window
is what speculation needs: a verification step feeds the matcher up to
``num_speculative_tokens`` draft tokens ahead of what the target model has confirmed, and the
rejected tail is rolled back. The reference sizes that window for its grammar back end as
``max(num_speculative_tokens, suffix_speculative_tokens)`` because suffix drafts can be longer
than the speculator's (arctic_inference/vllm/structured_output.py:29-39);
:func:`rollback_window` is the same rule.

Built in:

* :class:`ChoiceGrammar` -- the output is exactly one of a list of token sequences
  (``SamplingParams.guided_choice``), a trie over the tokenised choices.
* :class:`TokenSetGrammar` -- every token comes from a fixed set, up to a length
  (digits-only answers and the like).
* :class:`json_schema.CharMachineGrammar` over a compiled JSON schema -- compact JSON that
  conforms to the schema (``SamplingParams.guided_json``) -- or over a compiled regular
  expression (``SamplingParams.guided_regex``, :mod:`regex`).

Other matchers plug in by implementing :class:`Grammar`.
"""

from __future__ import annotations

from typing import Iterable, Optional, Sequence


def rollback_window(speculative_config) -> int:
    """Tokens a matcher must be able to take back in one step."""
    if speculative_config is None:
        return 0
    base = int(getattr(speculative_config, "num_speculative_tokens", 0) or 0)
    suffix = 0
    if getattr(speculative_config, "uses_suffix", False) or \
            getattr(speculative_config, "enable_suffix_decoding", False):
        suffix = int(getattr(speculative_config, "suffix_speculative_tokens", 0) or 0)
    return max(base, suffix)


class Grammar:
    """Matcher interface. States are opaque values; the matcher itself keeps a history of
    them so that :meth:`rollback` is a pop."""

    def allowed(self) -> Optional[Sequence[int]]:
        """Token ids allowed next, or None when every token is allowed."""
        raise NotImplementedError

    def accept(self, token: int) -> bool:
        """Advance over ``token``; False (and no change) if the grammar forbids it."""
        raise NotImplementedError

    def rollback(self, n: int) -> None:
        raise NotImplementedError

    @property
    def finished(self) -> bool:
        raise NotImplementedError

    # ------------------------------------------------------------------ speculation
    def validate_draft(self, draft: Iterable[int]) -> int:
        """Length of the longest prefix of ``draft`` the grammar accepts from its current
        state (the state is left unchanged)."""
        n = 0
        for t in draft:
            if self.finished or not self.accept(int(t)):
                break
            n += 1
        self.rollback(n)
        return n

    def allowed_along(self, draft: Sequence[int]) -> list:
        """``allowed()`` at the current state and after each token of a grammar-valid draft:
        one entry per verification row (len(draft) + 1)."""
        out = [self.allowed()]
        n = 0
        for t in draft:
            if self.finished or not self.accept(int(t)):
                break
            n += 1
            out.append(self.allowed())
        self.rollback(n)
        while len(out) < len(draft) + 1:
            out.append(None)      # rows behind an invalid draft token are discarded anyway
        return out


class _TrieNode:
    __slots__ = ("children", "terminal")

    def __init__(self):
        self.children: dict = {}
        self.terminal = False


class ChoiceGrammar(Grammar):
    """Exactly one of ``choices`` (token-id sequences). When a choice is a proper prefix of
    another one, ``eos_token_id`` ends the shorter one."""

    def __init__(self, choices: Sequence[Sequence[int]], eos_token_id: Optional[int] = None,
                 window: int = 0):
        if not choices or any(len(c) == 0 for c in choices):
            raise ValueError("guided choices must be non-empty token sequences")
        self.root = _TrieNode()
        for c in choices:
            node = self.root
            for t in c:
                node = node.children.setdefault(int(t), _TrieNode())
            node.terminal = True
        self.eos = eos_token_id
        self.window = window
        self._path = [self.root]      # history of states, last = current
        self._ended = False           # an explicit EOS closed a choice that is also a prefix

    @property
    def _node(self) -> _TrieNode:
        return self._path[-1]

    @property
    def finished(self) -> bool:
        n = self._node
        return self._ended or (n.terminal and not n.children)

    def allowed(self):
        if self.finished:
            return [self.eos] if self.eos is not None else []
        n = self._node
        toks = list(n.children)
        if n.terminal and self.eos is not None:
            toks.append(self.eos)
        return toks

    def accept(self, token: int) -> bool:
        if self.finished:
            return False
        n = self._node
        nxt = n.children.get(token)
        if nxt is not None:
            self._path.append(nxt)
            return True
        if n.terminal and self.eos is not None and token == self.eos:
            self._path.append(n)
            self._ended = True
            return True
        return False

    def rollback(self, n: int) -> None:
        if n <= 0:
            return
        if n >= len(self._path):
            raise ValueError("cannot roll back %d of %d tokens" % (n, len(self._path) - 1))
        del self._path[-n:]
        self._ended = False


class TokenSetGrammar(Grammar):
    """Every output token is in ``tokens``; the output ends after ``max_len`` tokens or, from
    ``min_len`` tokens on, with ``eos_token_id``."""

    def __init__(self, tokens: Iterable[int], max_len: int, min_len: int = 1,
                 eos_token_id: Optional[int] = None):
        self.tokens = sorted({int(t) for t in tokens})
        if not self.tokens or max_len < 1:
            raise ValueError("need a non-empty token set and max_len >= 1")
        self._set = set(self.tokens)
        self.max_len, self.min_len, self.eos = max_len, min_len, eos_token_id
        self._n = 0
        self._ended_at: Optional[int] = None

    @property
    def finished(self) -> bool:
        return self._ended_at is not None or self._n >= self.max_len

    def allowed(self):
        if self.finished:
            return [self.eos] if self.eos is not None else []
        if self.eos is not None and self._n >= self.min_len:
            return self.tokens + [self.eos]
        return self.tokens

    def accept(self, token: int) -> bool:
        if self.finished:
            return False
        if token in self._set:
            self._n += 1
            return True
        if self.eos is not None and token == self.eos and self._n >= self.min_len:
            self._n += 1
            self._ended_at = self._n
            return True
        return False

    def rollback(self, n: int) -> None:
        if n <= 0:
            return
        if n > self._n:
            raise ValueError("cannot roll back %d of %d tokens" % (n, self._n))
        self._n -= n
        if self._ended_at is not None and self._n < self._ended_at:
            self._ended_at = None


def build_grammar(params, tokenizer, eos_token_id, speculative_config=None) -> Optional[Grammar]:
    """The matcher a request's sampling parameters ask for, or None."""
    g = getattr(params, "grammar", None)
    if g is not None:
        return g
    schema = getattr(params, "guided_json", None)
    if schema is not None:
        from .json_schema import JsonSchemaGrammar, Vocabulary, compile_schema
        size = getattr(tokenizer, "vocab_size", None) or len(tokenizer)
        return JsonSchemaGrammar(compile_schema(schema), Vocabulary.from_tokenizer(tokenizer, size),
                                 eos_token_id)
    pattern = getattr(params, "guided_regex", None)
    if pattern is not None:
        from .json_schema import CharMachineGrammar, Vocabulary
        from .regex import compile_regex
        size = getattr(tokenizer, "vocab_size", None) or len(tokenizer)
        return CharMachineGrammar(compile_regex(pattern), Vocabulary.from_tokenizer(tokenizer, size),
                                  eos_token_id)
    choices = getattr(params, "guided_choice", None)
    if not choices:
        return None
    seqs = []
    for c in choices:
        if isinstance(c, str):
            try:
                ids = tokenizer.encode(c, add_special_tokens=False)
            except TypeError:
                ids = tokenizer.encode(c)
            ids = list(ids["input_ids"]) if isinstance(ids, dict) else list(ids)
        else:
            ids = [int(t) for t in c]
        seqs.append(ids)
    return ChoiceGrammar(seqs, eos_token_id, window=rollback_window(speculative_config))
