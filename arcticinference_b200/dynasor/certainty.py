"""Certainty bookkeeping of the early-exit controller: extracting the probed answer, deciding
whether the last few probes agree, and summary statistics over a set of answers.
(reference: arctic_inference/dynasor/cot.py:17-50, entropy.py:23-250.)
"""

from __future__ import annotations

import math
from typing import Any, Optional, Sequence

from .math_equal import math_equal

UNCERTAIN_WORDS = ("wait", "hold", "but", "okay", "no", "hmm")
DEFAULT_PROBE_SUFFIX = ("... Oh, I suddenly got the answer to the whole problem, "
                        "**Final Answer**\n\n\\[ \\boxed{")
SYSTEM_PROMPT = "You are a helpful assistant."


def obtain_answer(s: str) -> str:
    """Text up to the first unpaired ``}``: the content of the ``\\boxed{`` the probe left
    open. Empty when the brace never closes."""
    depth = 0
    for i, c in enumerate(s):
        if c == "{":
            depth += 1
        elif c == "}":
            if depth == 0:
                return s[:i]
            depth -= 1
    return ""


def is_certain_answer(probe_text: str, uncertain_words: Sequence[str] = UNCERTAIN_WORDS) -> bool:
    low = probe_text.lower()
    return not any(w in low for w in uncertain_words)


def has_value(x: Any) -> bool:
    if x is None:
        return False
    if isinstance(x, str):
        return len(x.strip()) > 0
    if isinstance(x, (list, tuple, dict, set)):
        return len(x) > 0
    return True


def count_not_empty(answers: Sequence) -> int:
    return sum(1 for a in answers if has_value(a))


def equal_group(answers: Sequence) -> bool:
    """All answers mathematically equal to the first one."""
    if not answers:
        return False
    return all(math_equal(answers[0], a) for a in answers[1:])


def group_counts(answers: Sequence) -> list:
    """Sizes of the equivalence classes of ``answers`` under ``math_equal``."""
    reps, counts = [], []
    for a in answers:
        for i, r in enumerate(reps):
            if math_equal(r, a):
                counts[i] += 1
                break
        else:
            reps.append(a)
            counts.append(1)
    return counts


def entropy(probs: Sequence[float]) -> float:
    return -sum(p * math.log(p) for p in probs if p > 0)


def item_entropy(answers: Sequence) -> float:
    c = group_counts([a for a in answers if has_value(a)])
    tot = sum(c)
    return entropy([x / tot for x in c]) if tot else 0.0


def majority_voting(answers: Sequence) -> Optional[Any]:
    reps, counts = [], []
    for a in answers:
        if not has_value(a):
            continue
        for i, r in enumerate(reps):
            if math_equal(r, a):
                counts[i] += 1
                break
        else:
            reps.append(a)
            counts.append(1)
    return reps[max(range(len(reps)), key=counts.__getitem__)] if reps else None


def should_early_exit(probe_answers: Sequence[str], probe_responses: Sequence[str],
                      certainty_window: int,
                      uncertain_words: Sequence[str] = UNCERTAIN_WORDS) -> bool:
    """True when the last ``certainty_window`` probes gave a non-empty, mutually equal answer
    and none of those probe continuations contains a hesitation word."""
    if certainty_window <= 0 or len(probe_answers) < certainty_window:
        return False
    last_a = list(probe_answers[-certainty_window:])
    last_r = list(probe_responses[-certainty_window:])
    return (count_not_empty(last_a) == certainty_window and equal_group(last_a)
            and all(is_certain_answer(r, uncertain_words) for r in last_r))


def format_probe_prompt(prompt: str, generated: str, suffix: str = DEFAULT_PROBE_SUFFIX,
                        template: Optional[str] = None) -> str:
    """Raw-completions prompt of a probe: the conversation so far, the reasoning generated so
    far, and the suffix that makes the model blurt out its current answer. ``template`` has
    the fields {system}, {prompt}, {generated}, {suffix}; the default is the DeepSeek-R1
    layout the reference hard-codes (cot.py:26-29)."""
    template = template or ("<｜begin▁of▁sentence｜>{system}<｜User｜>{prompt}<｜Assistant｜>"
                            "<think>\n{generated} {suffix}")
    return template.format(system=SYSTEM_PROMPT, prompt=prompt, generated=generated, suffix=suffix)


def formalize_final_response(generated_text: str, answer: str) -> str:
    close = "" if "</think>" in generated_text else "</think>\n"
    lead = "\n\n... " if close == "" else "\n\n..."
    return "%s%sOh, I have got the answer to the whole problem\n**Final Answer:**\n\\[\n \\boxed{%s}\n\\]" % (
        lead, close + (" " if close else ""), answer)
