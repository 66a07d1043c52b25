"""End-to-end checks of the engine on a GPU: the CUDA forward pass against the
PyTorch restatement of the same model, and generation through the public API."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams, ops
from arcticinference_b200.config import EngineArgs

pytestmark = pytest.mark.gpu


def _copy_weights(src, dst):
    for (n1, t1), (n2, t2) in zip(src.named_tensors(), dst.named_tensors()):
        assert n1 == n2
        t2.copy_(t1.to(t2.device))


def _engine_pair(model, **kw):
    gpu = LLM(model=model, device="cuda:0", num_gpu_blocks_override=128, block_size=16,
              max_model_len=1024, **kw)
    cpu = LLM(model=model, device="cpu", num_gpu_blocks_override=128, block_size=16,
              max_model_len=1024, **kw)
    _copy_weights(gpu.engine.runner.model, cpu.engine.runner.model)
    return gpu, cpu


@pytest.mark.parametrize("model", ["llama-tiny", "llama-tiny-swiftkv"])
def test_forward_matches_reference(model):
    gpu, cpu = _engine_pair(model)
    prompts = [list(range(3, 150)), [9, 8, 7, 6], list(range(200, 260))]
    hs = []
    for llm in (gpu, cpu):
        eng = llm.engine
        for p in prompts:
            eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
        out = eng.scheduler.schedule()
        batch, rows = eng.runner.prepare(out)
        with torch.inference_mode():
            h = eng.runner.model.forward(batch, eng.runner.kv)
            logits = eng.runner.model.compute_logits(h)
        hs.append(logits.float().cpu())
    ops.check_status()
    err = (hs[0] - hs[1]).abs().max().item()
    assert err < 0.08 * max(1.0, hs[1].abs().max().item()), err


@pytest.mark.parametrize("model", ["llama-tiny", "llama-tiny-swiftkv"])
def test_generate_matches_reference_tokens(model):
    gpu, cpu = _engine_pair(model)
    prompts = [{"prompt_token_ids": list(range(5, 90))}, {"prompt_token_ids": [4, 4, 8, 15, 16]}]
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    a = gpu.generate(prompts, sp)
    b = cpu.generate(prompts, sp)
    ops.check_status()
    # greedy tokens agree except where bf16 rounding flips a near-tie; require the first
    # token of each request and most of the rest to match
    match = total = 0
    for x, y in zip(a, b):
        assert x.outputs[0].token_ids[0] == y.outputs[0].token_ids[0]
        for p, q in zip(x.outputs[0].token_ids, y.outputs[0].token_ids):
            match += int(p == q)
            total += 1
    assert match >= 0.7 * total


def _first_step_logits(llm, prompt, sp):
    """Generate and return (outputs, logits of the first sampled position)."""
    model = llm.engine.runner.model
    seen = []
    orig = model.compute_logits

    def spy(hidden, fp32=False):
        out = orig(hidden, fp32=fp32)
        seen.append(out.float().clone())
        return out

    model.compute_logits = spy
    try:
        outs = llm.generate([prompt], sp)
    finally:
        model.compute_logits = orig
    return outs, seen[0][0]


def test_chunked_prefill_equals_single_shot():
    # a tiny random model has near-ties in its logits, so the comparison is on the logits
    # themselves (and on the arg-max only where it is decided by a clear margin)
    sp = SamplingParams(temperature=0, max_tokens=5, ignore_eos=True)
    prompt = {"prompt_token_ids": [(7 * i) % 1000 + 1 for i in range(700)]}
    kw = dict(model="llama-tiny", device="cuda:0", num_gpu_blocks_override=128, block_size=16,
              max_model_len=1024, enforce_eager=True)
    a, la = _first_step_logits(LLM(max_num_batched_tokens=4096, **kw), prompt, sp)
    b, lb = _first_step_logits(LLM(max_num_batched_tokens=256, **kw), prompt, sp)
    ops.check_status()
    scale = float(la.abs().max())
    assert float((la - lb).abs().max()) < 0.03 * scale + 0.03
    top2 = torch.topk(la, 2).values
    if float(top2[0] - top2[1]) > 0.06 * scale + 0.06:
        assert a[0].outputs[0].token_ids[0] == b[0].outputs[0].token_ids[0]


def test_prefix_cache_hit_gives_same_tokens():
    llm = LLM(model="llama-tiny", device="cuda:0", num_gpu_blocks_override=128, block_size=16,
              max_model_len=1024)
    sp = SamplingParams(temperature=0, max_tokens=5, ignore_eos=True)
    p = {"prompt_token_ids": list(range(10, 110))}
    a = llm.generate([p], sp)
    b = llm.generate([p], sp)
    ops.check_status()
    assert b[0].num_cached_tokens == 96
    assert a[0].outputs[0].token_ids[0] == b[0].outputs[0].token_ids[0]


def test_sleep_wake_roundtrip():
    llm = LLM(model="llama-tiny", device="cuda:0", num_gpu_blocks_override=64, block_size=16,
              max_model_len=512, enable_sleep_mode=True)
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    p = {"prompt_token_ids": list(range(10, 60))}
    before = llm.generate([p], sp)[0].outputs[0].token_ids
    for level in (1, 2):
        llm.sleep(level)
        llm.wake_up(["weights"])
        llm.wake_up(["kv_cache"])
        after = llm.generate([p], sp)[0].outputs[0].token_ids
        assert after == before
    ops.check_status()


@pytest.mark.parametrize("model", ["llama-small", "llama-tiny-swiftkv"])
def test_cuda_graph_decode_matches_eager(model):
    sp = SamplingParams(temperature=0, max_tokens=12, ignore_eos=True)
    prompts = [{"prompt_token_ids": list(range(5, 5 + n))} for n in (40, 7, 300, 65, 130)]
    kw = dict(model=model, device="cuda:0", num_gpu_blocks_override=256, block_size=16,
              max_model_len=1024)
    eager = LLM(enforce_eager=True, **kw)
    a = eager.generate(prompts, sp)
    graphed = LLM(enforce_eager=False, **kw)
    b = graphed.generate(prompts, sp)
    ops.check_status()
    assert graphed.engine.runner.graph_replays > 0
    assert eager.engine.runner.graph_replays == 0
    for x, y in zip(a, b):
        assert x.outputs[0].token_ids == y.outputs[0].token_ids


@pytest.mark.parametrize("spec", [
    {"method": "suffix"},
    {"method": "arctic", "model": "random", "num_speculative_tokens": 3,
     "enable_suffix_decoding": True},
])
def test_speculative_decoding_preserves_output_on_gpu(spec):
    kw = dict(model="llama-small", device="cuda:0", num_gpu_blocks_override=256, block_size=16,
              max_model_len=1024)
    prompts = [{"prompt_token_ids": [5, 6, 7, 8, 9, 10] * 8}, {"prompt_token_ids": list(range(40, 75))}]
    sp = SamplingParams(temperature=0, max_tokens=32, ignore_eos=True)
    base = LLM(**kw).generate(prompts, sp)
    llm = LLM(speculative_config=spec, **kw)
    outs = llm.generate(prompts, sp)
    ops.check_status()
    assert llm.engine.stats["draft_tokens"] > 0
    match = sum(int(a == b) for x, y in zip(base, outs)
                for a, b in zip(x.outputs[0].token_ids, y.outputs[0].token_ids))
    total = sum(len(x.outputs[0].token_ids) for x in base)
    # Verification scores several tokens of a request in one pass, which rounds differently from
    # one token at a time; the random model's top logits lie close together, so a near-tie can
    # fall the other way and the two continuations part from there (exact equality of
    # speculative and plain greedy decoding is asserted on the CPU path, where both round
    # alike). Here: the first tokens agree and the runs do not part at once.
    assert all(x.outputs[0].token_ids[0] == y.outputs[0].token_ids[0] for x, y in zip(base, outs))
    assert match >= 0.25 * total
    assert all(len(o.outputs[0].token_ids) == 32 for o in outs)


def test_forest_cascade_matches_plain_decode():
    """Parallel samples of one long prompt share its KV blocks: the cascade reads them once."""
    kw = dict(model="llama-small", device="cuda:0", num_gpu_blocks_override=512, block_size=16,
              max_model_len=1024)
    shared = list(range(7, 7 + 400))
    prompts = [{"prompt_token_ids": shared + [900 + i]} for i in range(10)]
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    plain = LLM(**kw).generate(prompts, sp)
    fca = LLM(forest_cascade_attn_configs="{}", **kw)
    fca.generate(prompts[:1], sp)          # fills the prefix cache: later requests share blocks
    outs = fca.generate(prompts, sp)
    ops.check_status()
    assert fca.engine.runner.cascade_steps > 0
    match = sum(int(a == b) for x, y in zip(plain, outs)
                for a, b in zip(x.outputs[0].token_ids, y.outputs[0].token_ids))
    assert match >= 0.8 * 60


def test_run_ahead_scheduling_changes_nothing():
    sp = [SamplingParams(temperature=0, max_tokens=n, ignore_eos=True) for n in (20, 33, 5, 48)]
    prompts = [{"prompt_token_ids": [(11 * i + j) % 997 + 1 for i in range(40 + 30 * j)]} for j in range(4)]
    kw = dict(model="llama-tiny", device="cuda:0", num_gpu_blocks_override=256, block_size=16,
              max_model_len=512)
    outs = {}
    for mode in (False, True):
        llm = LLM(async_scheduling=mode, **kw)
        outs[mode] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if mode:
            assert llm.engine.stats["run_ahead_steps"] > 20 and llm.engine.runner.graph_replays > 20
    ops.check_status()
    assert outs[False] == outs[True]
    # token-dependent stop in the middle of a run-ahead stretch
    stop = outs[False][1][10]
    sp2 = SamplingParams(temperature=0, max_tokens=48, stop_token_ids=[stop])
    a = LLM(async_scheduling=False, **kw).generate(prompts, sp2)
    b = LLM(async_scheduling=True, **kw).generate(prompts, sp2)
    assert [o.outputs[0].token_ids for o in a] == [o.outputs[0].token_ids for o in b]
    assert [o.outputs[0].finish_reason for o in a] == [o.outputs[0].finish_reason for o in b]


def test_async_engine_on_the_default_device_streams_tokens():
    """The streaming front end with the device given as plain "cuda" (what the servers and
    the trace replay use): its loop thread must come up on the current device, and a
    request must stream to completion."""
    import asyncio
    from arcticinference_b200.engine.async_llm import AsyncLLM
    llm = AsyncLLM.from_engine_args(EngineArgs(model="llama-tiny", max_model_len=256,
                                               num_gpu_blocks_override=64)).start()
    try:
        assert llm.engine.device.type == "cuda"

        async def run():
            sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
            outs = await asyncio.wait_for(
                asyncio.gather(*[llm.generate_final(list(range(5 + i, 40 + i)), sp)
                                 for i in range(3)]), timeout=120)
            return [len(o.outputs[0].token_ids) for o in outs]

        assert asyncio.run(run()) == [12, 12, 12]
    finally:
        llm.shutdown()
    ops.check_status()


def test_run_ahead_over_chunked_prompts_changes_nothing():
    """Prompt chunks and completing prompts run ahead too: long prompts cut into 64-token
    chunks that share steps with other requests' decodes give the same tokens with run-ahead
    stepping on and off, and nearly every step is queued behind its predecessor."""
    prompts = [{"prompt_token_ids": [(7 * i + 3 * j) % 997 + 1 for i in range(n)]}
               for j, n in enumerate((300, 12, 150, 70))]
    sp = [SamplingParams(temperature=0, max_tokens=n, ignore_eos=True) for n in (10, 40, 1, 25)]
    kw = dict(model="llama-tiny", device="cuda:0", num_gpu_blocks_override=256, block_size=16,
              max_model_len=512, max_num_batched_tokens=64)
    outs, steps = {}, {}
    for mode in (False, True):
        llm = LLM(async_scheduling=mode, **kw)
        outs[mode] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        steps[mode] = llm.engine.stats["steps"]
        if mode:
            assert llm.engine.stats["run_ahead_steps"] >= steps[mode] - 3
    ops.check_status()
    assert outs[False] == outs[True] and steps[False] == steps[True]


def test_logprobs_on_gpu_match_the_cpu_path():
    """Same weights on both devices (random weights are drawn by the device's own generator, so
    they are copied across): prompt and output log-probabilities agree to bf16 accuracy."""
    import math
    gpu, cpu = _engine_pair("llama-tiny")
    prompt = [{"prompt_token_ids": [(5 * i) % 991 + 2 for i in range(48)]}]
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True, logprobs=2, prompt_logprobs=0)
    g = gpu.generate(prompt, sp)[0]
    c = cpu.generate(prompt, sp)[0]
    ops.check_status()
    assert len(g.prompt_logprobs) == 48 and g.prompt_logprobs[0] is None
    assert all(math.isclose(a, b, abs_tol=0.12) for a, b in zip(g.prompt_logprobs[1:], c.prompt_logprobs[1:]))
    assert len(g.outputs[0].logprobs) == 6 and len(g.outputs[0].top_logprobs[0]) == 2
    assert math.isclose(g.outputs[0].logprobs[0], c.outputs[0].logprobs[0], abs_tol=0.12)


@pytest.mark.parametrize("scheme", ["channel", "block"])
def test_fp8_engine_matches_the_cpu_path(scheme):
    """fp8 linears (per-token / per-feature scales with the fused quantising norm and SiLU
    kernels, or 128 x 128 blocks) against the PyTorch restatement with the same quantised
    weights: first-step logits agree to the accuracy of the activations' fp8 rounding."""
    kw = dict(model="llama-small", num_gpu_blocks_override=128, block_size=16, max_model_len=1024)
    gpu = LLM(device="cuda:0", **kw)
    cpu = LLM(device="cpu", **kw)
    _copy_weights(gpu.engine.runner.model, cpu.engine.runner.model)
    from arcticinference_b200.models.quant import quantize_model_fp8
    for llm in (gpu, cpu):
        quantize_model_fp8(llm.engine.runner.model, prefill_shadow=False, scheme=scheme)
    prompts = [list(range(3, 150)), [9, 8, 7, 6], list(range(200, 260))]
    hs = []
    for llm in (gpu, cpu):
        eng = llm.engine
        for p in prompts:
            eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
        out = eng.scheduler.schedule()
        batch, rows = eng.runner.prepare(out)
        with torch.inference_mode():
            h = eng.runner.model.forward(batch, eng.runner.kv)
            logits = eng.runner.model.compute_logits(h)
        hs.append(logits.float().cpu())
    ops.check_status()
    err = (hs[0] - hs[1]).abs().max().item()
    assert err < 0.1 * max(1.0, hs[1].abs().max().item()), err


@pytest.mark.gpu
def test_programmatic_dependent_launch_gives_the_same_tokens():
    """AB200_PDL=1 launches the serving kernels with programmatic stream serialisation (set-up
    and the first weight tiles of a kernel overlap the tail of the one before it). The switch is
    read once per process, so the opted-in run is a child process; greedy tokens must agree."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import json, sys; sys.path.insert(0, %r)\n"
        "from arcticinference_b200 import LLM, SamplingParams, ops\n"
        "llm = LLM(model='llama-small', device='cuda:0', max_model_len=1024, num_gpu_blocks_override=256,"
        " quantization='fp8')\n"
        "outs = llm.generate([{'prompt_token_ids': list(range(1, 200))}, {'prompt_token_ids': [5, 6, 7]}],"
        " SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))\n"
        "ops.check_status()\n"
        "print('TOKENS ' + json.dumps([o.outputs[0].token_ids for o in outs]))\n" % root)
    toks = {}
    for flag in ("0", "1"):
        env = dict(os.environ, AB200_PDL=flag, ARCTIC_B200_NO_AUTOBUILD="1")
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                             timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        line = [l for l in out.stdout.splitlines() if l.startswith("TOKENS ")][-1]
        toks[flag] = json.loads(line[len("TOKENS "):])
    same = sum(int(a == b) for x, y in zip(toks["0"], toks["1"]) for a, b in zip(x, y))
    assert [t[0] for t in toks["0"]] == [t[0] for t in toks["1"]]
    assert same >= 0.75 * sum(len(t) for t in toks["0"])
