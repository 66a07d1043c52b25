"""The early-exit loop, independent of transport.

``DynasorController.run`` consumes a stream of generated text chunks. Every
``probe_interval`` chunks it launches (concurrently with generation) a *probe*: a short
completion of "prompt + reasoning so far + probing suffix". When the last
``certainty_window`` probes agree on a non-empty answer without hesitation words, generation
is cut and a closing text with the agreed answer is emitted. The HTTP proxy and the
in-process server both drive this class (reference: arctic_inference/dynasor/
openai_server.py:190-350, cot.py:53-150).
"""

from __future__ import annotations

import asyncio
from dataclasses import dataclass, field
from typing import AsyncIterator, Awaitable, Callable, Optional

from .certainty import (DEFAULT_PROBE_SUFFIX, formalize_final_response, obtain_answer,
                        should_early_exit)


@dataclass
class DynasorStats:
    chunks: int = 0
    probes: int = 0
    early_exit: bool = False
    answer: Optional[str] = None
    probe_answers: list = field(default_factory=list)


class DynasorController:
    def __init__(self, probe_fn: Callable[[str], Awaitable[str]], probe_interval: int = 32,
                 certainty_window: int = 3, probe_suffix: str = DEFAULT_PROBE_SUFFIX):
        """``probe_fn(generated_so_far)`` returns the probe's continuation text."""
        self.probe_fn = probe_fn
        self.probe_interval = max(1, probe_interval)
        self.certainty_window = certainty_window
        self.probe_suffix = probe_suffix
        self.stats = DynasorStats()

    async def run(self, chunks: AsyncIterator[str]) -> AsyncIterator[str]:
        st = self.stats
        generated = ""
        answers, responses = [], []
        probe: Optional[asyncio.Task] = None
        want_probe = False
        try:
            async for text in chunks:
                generated += text
                st.chunks += 1
                yield text
                if st.chunks % self.probe_interval == 0:
                    want_probe = True
                if probe is not None and probe.done():
                    resp = probe.result()
                    probe = None
                    answers.append(obtain_answer(resp))
                    responses.append(resp)
                    st.probe_answers = list(answers)
                    if should_early_exit(answers, responses, self.certainty_window):
                        st.early_exit = True
                        st.answer = answers[-1]
                        yield formalize_final_response(generated, answers[-1])
                        return
                if want_probe and probe is None:
                    want_probe = False
                    st.probes += 1
                    probe = asyncio.ensure_future(self.probe_fn(generated))
        finally:
            if probe is not None:
                probe.cancel()
            aclose = getattr(chunks, "aclose", None)
            if aclose is not None:
                await aclose()
