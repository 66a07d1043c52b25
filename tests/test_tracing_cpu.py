"""Tracing: ranges are free when off, collected when a tracer is installed, and the engine's
step phases show up in the Chrome trace."""

import json

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.utils import tracing


def test_ranges_off_and_on(tmp_path):
    with tracing.trace_range("nothing"):
        pass
    with tracing.Tracer() as t:
        with tracing.trace_range("outer", k=1):
            with tracing.trace_range("inner"):
                pass
    names = [e["name"] for e in t.events]
    assert names == ["inner", "outer"] and t.events[1]["args"] == {"k": 1}
    assert t.events[1]["dur"] >= t.events[0]["dur"]
    out = tmp_path / "trace.json"
    t.dump(str(out))
    assert len(json.load(open(out))["traceEvents"]) == 2


def test_engine_phases_are_traced():
    llm = LLM(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16, max_model_len=128)
    with tracing.Tracer() as t:
        llm.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    tot = t.totals()
    assert {"prepare", "forward", "sample", "sync_tokens"} <= set(tot)
    assert tot["forward"][1] == 4
