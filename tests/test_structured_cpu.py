"""Grammar-constrained outputs: the matchers, their take-back window, and the engine path
(with and without speculative decoding)."""

import pytest

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import SpeculativeConfig
from arcticinference_b200.structured import (ChoiceGrammar, TokenSetGrammar, build_grammar,
                                             rollback_window)


def test_choice_grammar_walks_and_rolls_back():
    g = ChoiceGrammar([[5, 6, 7], [5, 9], [4]], eos_token_id=2)
    assert sorted(g.allowed()) == [4, 5]
    assert not g.accept(6) and g.accept(5)
    assert sorted(g.allowed()) == [6, 9]
    assert g.validate_draft([6, 7, 8]) == 2          # state unchanged afterwards
    assert sorted(g.allowed()) == [6, 9]
    rows = g.allowed_along([6, 7])
    assert [sorted(r) for r in rows] == [[6, 9], [7], [2]]
    assert g.accept(6) and g.accept(7) and g.finished
    g.rollback(2)
    assert not g.finished and g.accept(9) and g.finished
    with pytest.raises(ValueError):
        g.rollback(5)


def test_choice_that_is_a_prefix_ends_with_eos():
    g = ChoiceGrammar([[5], [5, 6]], eos_token_id=2)
    assert g.accept(5) and not g.finished
    assert sorted(g.allowed()) == [2, 6]
    assert g.accept(2) and g.finished
    g.rollback(1)
    assert not g.finished and g.accept(6) and g.finished


def test_token_set_grammar():
    g = TokenSetGrammar([7, 8, 9], max_len=3, min_len=2, eos_token_id=2)
    assert g.allowed() == [7, 8, 9] and not g.accept(2)
    assert g.accept(7) and g.accept(9)
    assert g.allowed() == [7, 8, 9, 2]
    assert g.validate_draft([8, 8]) == 1
    assert g.accept(2) and g.finished
    g.rollback(2)
    assert not g.finished and g.accept(8) and g.accept(8) and g.finished


def test_rollback_window_follows_the_longer_drafter():
    assert rollback_window(None) == 0
    arctic = SpeculativeConfig(method="arctic", model="random", num_speculative_tokens=3)
    assert rollback_window(arctic) == 3
    hybrid = SpeculativeConfig(method="arctic", model="random", num_speculative_tokens=3,
                               enable_suffix_decoding=True)
    assert rollback_window(hybrid) == max(3, hybrid.suffix_speculative_tokens)
    assert rollback_window(hybrid) > 3


CHOICES = ["yes", "no", "maybe so"]


@pytest.mark.parametrize("spec", [None, {"method": "suffix"},
                                  {"method": "arctic", "model": "random",
                                   "num_speculative_tokens": 3}])
def test_engine_output_is_one_of_the_choices(spec):
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64,
              speculative_config=spec)
    prompts = [{"prompt_token_ids": list(range(10 + i, 40 + i))} for i in range(6)]
    params = [SamplingParams(temperature=1.0 if i % 2 else 0.0, seed=i, max_tokens=32,
                             guided_choice=CHOICES) for i in range(6)]
    outs = llm.generate(prompts, params)
    texts = [o.outputs[0].text for o in outs]
    assert all(t in CHOICES for t in texts), texts
    assert all(o.outputs[0].finish_reason == "stop" for o in outs)
    # unconstrained requests in the same batch are left alone
    mixed = llm.generate(prompts[:2], [SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True),
                                      SamplingParams(temperature=0.0, max_tokens=8,
                                                     guided_choice=["no"])])
    assert len(mixed[0].outputs[0].token_ids) == 8 and mixed[1].outputs[0].text == "no"


def test_parallel_samples_get_their_own_matcher():
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64)
    tok = llm.engine.tokenizer
    g = build_grammar(SamplingParams(guided_choice=CHOICES), tok, 2)
    sp = SamplingParams(n=3, temperature=1.0, seed=3, max_tokens=16, grammar=g)
    out = llm.generate([{"prompt_token_ids": list(range(5, 30))}], sp)[0]
    assert len(out.outputs) == 3 and all(c.text in CHOICES for c in out.outputs)
    assert not g.finished          # the caller's object was copied, not consumed


# ------------------------------------------------------------------------------ JSON schema
SCHEMA = {
    "type": "object",
    "properties": {
        "name": {"type": "string", "maxLength": 6},
        "age": {"type": "integer"},
        "score": {"type": "number"},
        "tags": {"type": "array", "items": {"type": "string", "maxLength": 3}, "maxItems": 2},
        "ok": {"type": "boolean"},
        "color": {"enum": ["red", "green", 3, None]},
        "inner": {"$ref": "#/$defs/Point"},
    },
    "$defs": {"Point": {"type": "object",
                        "properties": {"x": {"type": "integer"},
                                       "y": {"type": "array", "items": {"type": "number"},
                                             "minItems": 1, "maxItems": 2}}}},
}


def _conforms(doc):
    assert set(doc) == {"name", "age", "score", "tags", "ok", "color", "inner"}
    assert isinstance(doc["name"], str) and len(doc["name"]) <= 6
    assert isinstance(doc["age"], int) and not isinstance(doc["age"], bool)
    assert isinstance(doc["score"], (int, float))
    assert isinstance(doc["tags"], list) and len(doc["tags"]) <= 2
    assert isinstance(doc["ok"], bool) and doc["color"] in ("red", "green", 3, None)
    assert isinstance(doc["inner"]["x"], int) and 1 <= len(doc["inner"]["y"]) <= 2


def test_schema_matcher_accepts_and_rejects():
    from arcticinference_b200.structured.json_schema import CompiledSchema
    c = CompiledSchema(SCHEMA)
    good = ['{"name":"ab","age":-12,"score":1.5e3,"tags":[],"ok":true,"color":"red",'
            '"inner":{"x":0,"y":[1]}}',
            '{"name":"a\\"b","age":0,"score":0,"tags":["x","y"],"ok":false,"color":null,'
            '"inner":{"x":7,"y":[1.0,2]}}']
    for g in good:
        assert c.validate(g), g
    bad = [good[0].replace('"ab"', '"abcdefg"'), good[0].replace("-12", "012"),
           good[0].replace('"red"', '"blue"'), good[0].replace("[1]", "[]"),
           good[0].replace("[]", '["a","b","c"]'), good[0][:-1], '{"age":1}']
    for b in bad:
        assert not c.validate(b), b
    with pytest.raises(ValueError):
        CompiledSchema({"type": "string", "pattern": "a+"})       # not anchored


def test_schema_grammar_on_tokens_with_rollback():
    from arcticinference_b200.structured.json_schema import (JsonSchemaGrammar, Vocabulary,
                                                             compile_schema)
    # a vocabulary with multi-character tokens that straddle syntax
    words = [None, None, None, '{"', 'x', '":', '1', '2', '}', '":1', '2}', '"', ',', 'x":']
    g = JsonSchemaGrammar(compile_schema({"type": "object", "properties": {"x": {"type": "integer"}}}),
                          Vocabulary(words), eos_token_id=2)
    tid = {w: i for i, w in enumerate(words) if w}
    assert sorted(g.allowed()) == [tid['{"']]
    assert g.accept(tid['{"'])
    assert sorted(g.allowed()) == sorted([tid['x'], tid['x":']])
    assert g.validate_draft([tid['x":'], tid['1'], tid['2}'], tid['1']]) == 3
    assert g.accept(tid['x']) and g.accept(tid['":1'])
    assert sorted(g.allowed()) == sorted([tid['1'], tid['2'], tid['}'], tid['2}']])
    assert g.accept(tid['2}']) and g.finished
    g.rollback(1)
    assert not g.finished and g.accept(tid['}']) and g.finished


@pytest.mark.parametrize("spec", [None, {"method": "suffix"}])
def test_engine_emits_documents_that_conform(spec):
    import json
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=512, num_gpu_blocks_override=128,
              speculative_config=spec)
    prompts = [{"prompt_token_ids": list(range(20 + i, 50 + i))} for i in range(4)]
    params = [SamplingParams(temperature=0.9 if i else 0.0, seed=10 + i, max_tokens=400,
                             guided_json=SCHEMA) for i in range(4)]
    for o in llm.generate(prompts, params):
        assert o.outputs[0].finish_reason == "stop", o.outputs[0].text
        _conforms(json.loads(o.outputs[0].text))


def test_unions_and_optional_properties():
    from arcticinference_b200.structured.json_schema import CompiledSchema
    c = CompiledSchema({"type": "object", "required": ["b"], "properties": {
        "a": {"type": "integer"}, "b": {"type": ["string", "null"]},
        "c": {"anyOf": [{"type": "number"}, {"type": "array", "items": {"type": "integer"}}]}}})
    for t in ['{"a":1,"b":"x","c":2.5}', '{"b":null}', '{"b":"q","c":[1,2]}', '{"a":0,"b":null}']:
        assert c.validate(t), t
    for t in ['{"a":1}', '{}', '{"b":1}', '{"c":1,"b":null}', '{"b":null,}', '{,"b":null}']:
        assert not c.validate(t), t
    # readings that share a prefix stay alive side by side: 12 is an integer and a number
    u = CompiledSchema({"anyOf": [{"type": "integer"}, {"type": "number"}, {"const": "n/a"}]})
    assert u.validate("12") and u.validate("1.5e2") and u.validate('"n/a"')
    assert not u.validate('"x"') and not u.validate("1.")
    st = u.advance_text(u.start(), "12")
    assert len(st) == 2 and u.complete(st) and not u.exhausted(st)


def test_engine_with_optional_fields_and_unions():
    import json
    schema = {"type": "object", "required": ["kind"], "properties": {
        "kind": {"enum": ["a", "b"]}, "n": {"type": ["integer", "null"]},
        "tags": {"type": "array", "items": {"enum": ["x", "y"]}, "maxItems": 3}}}
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=512, num_gpu_blocks_override=128)
    prompts = [{"prompt_token_ids": list(range(40 + i, 60 + i))} for i in range(5)]
    params = [SamplingParams(temperature=1.0, seed=i, max_tokens=200, guided_json=schema)
              for i in range(5)]
    seen = set()
    for o in llm.generate(prompts, params):
        doc = json.loads(o.outputs[0].text)
        assert doc["kind"] in ("a", "b") and set(doc) <= {"kind", "n", "tags"}
        assert doc.get("n") is None or isinstance(doc["n"], int)
        assert all(t in ("x", "y") for t in doc.get("tags", [])) and len(doc.get("tags", [])) <= 3
        seen.add(tuple(sorted(doc)))
    assert len(seen) >= 1


# ------------------------------------------------------------------------------------ regex
REGEX_CASES = {
    r"\d{3}-\d{4}": (["555-1234"], ["5555-123", "555-123", "a55-1234"]),
    r"(yes|no|maybe)( please)?": (["yes", "no please", "maybe"], ["yes  please", "y", ""]),
    r"[A-Z][a-z]+(, [A-Z][a-z]+)*\.": (["Hello.", "Hello, World."], ["hello.", "Hello,World."]),
    r"^-?(0|[1-9]\d*)(\.\d+)?$": (["0", "-12.50", "7"], ["01", "1.", "--1"]),
    r"[^abc\d]+x?": (["zzz", "qx"], ["a", "1", "zx1"]),
    r"a{2,3}b*?c+": (["aac", "aaabbcc"], ["ac", "aaaac", "aab"]),
    r"(?:ab)*": (["", "ab", "abab"], ["a", "aba"]),
    r"\w+@\w+\.(com|org)": (["me@x.org"], ["me@x.net", "@x.com"]),
}


def test_regex_compiler_agrees_with_re():
    import re
    from arcticinference_b200.structured.regex import CompiledRegex
    for pat, (good, bad) in REGEX_CASES.items():
        c = CompiledRegex(pat)
        for t in good:
            assert re.fullmatch(pat, t) and c.validate(t), (pat, t)
        for t in bad:
            assert not re.fullmatch(pat, t) and not c.validate(t), (pat, t)
    for pat in [r"(a", r"a)", r"*a", r"(?=a)b", r"a\1", r"[a", r"a{3,2}"]:
        with pytest.raises(ValueError):
            CompiledRegex(pat)
    c = CompiledRegex(r"ab?")
    st = c.advance_text(c.start(), "a")
    assert c.complete(st) and not c.exhausted(st)
    assert c.exhausted(c.advance_text(c.start(), "ab"))


@pytest.mark.parametrize("spec", [None, {"method": "suffix"}])
def test_engine_output_matches_the_expression(spec):
    import re
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64,
              speculative_config=spec)
    pat = r"(ID|REF)-\d{2,4}(/[a-f]{1,3})?"
    prompts = [{"prompt_token_ids": list(range(15 + i, 45 + i))} for i in range(5)]
    params = [SamplingParams(temperature=1.0 if i else 0.0, seed=i, max_tokens=40,
                             guided_regex=pat) for i in range(5)]
    for o in llm.generate(prompts, params):
        assert re.fullmatch(pat, o.outputs[0].text), o.outputs[0].text
        assert o.outputs[0].finish_reason == "stop"


def test_string_patterns_inside_a_schema():
    import json
    from arcticinference_b200.structured.json_schema import CompiledSchema
    schema = {"type": "object", "properties": {
        "id": {"type": "string", "pattern": "^[A-Z]{2}-\\d{3}$"},
        "date": {"type": "string", "pattern": "^\\d{4}-\\d{2}-\\d{2}$"}}}
    c = CompiledSchema(schema)
    assert c.validate('{"id":"AB-123","date":"2024-01-31"}')
    for t in ['{"id":"AB-12","date":"2024-01-31"}', '{"id":"ab-123","date":"2024-01-31"}',
              '{"id":"AB-123","date":"2024-1-31"}']:
        assert not c.validate(t), t
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64)
    outs = llm.generate([{"prompt_token_ids": list(range(9, 40))}] * 3,
                        [SamplingParams(temperature=1.0, seed=i, max_tokens=60, guided_json=schema)
                         for i in range(3)])
    import re
    for o in outs:
        doc = json.loads(o.outputs[0].text)
        assert re.fullmatch(r"[A-Z]{2}-\d{3}", doc["id"]) and re.fullmatch(r"\d{4}-\d{2}-\d{2}", doc["date"])


# ------------------------------------------------------------------ randomised schema check
def _random_schema(rng, depth=0):
    kinds = ["string", "integer", "number", "boolean", "null", "enum", "union"]
    if depth < 2:
        kinds += ["array", "object", "object"]
    k = rng.choice(kinds)
    if k == "string":
        return {"type": "string", "maxLength": rng.randint(0, 6)} if rng.random() < 0.7 else {"type": "string"}
    if k in ("integer", "number", "boolean", "null"):
        return {"type": k}
    if k == "enum":
        pool = ["a", "b c", 1, 2.5, True, None, 'q"uote']
        return {"enum": rng.sample(pool, rng.randint(1, 4))}
    if k == "union":
        return {"anyOf": [_random_schema(rng, depth + 1) for _ in range(rng.randint(2, 3))]}
    if k == "array":
        lo = rng.randint(0, 2)
        return {"type": "array", "items": _random_schema(rng, depth + 1), "minItems": lo,
                "maxItems": lo + rng.randint(0, 2)}
    names = rng.sample(["a", "b", "c", "d", "key with space"], rng.randint(1, 4))
    sch = {"type": "object", "properties": {n: _random_schema(rng, depth + 1) for n in names}}
    if rng.random() < 0.6:
        sch["required"] = [n for n in names if rng.random() < 0.5]
    return sch


def _random_instance(rng, sch):
    if "enum" in sch:
        return rng.choice(sch["enum"])
    if "anyOf" in sch:
        return _random_instance(rng, rng.choice(sch["anyOf"]))
    t = sch["type"]
    if t == "string":
        n = rng.randint(0, sch.get("maxLength", 8))
        return "".join(rng.choice('ab "\\/é\n7') for _ in range(n))
    if t == "integer":
        return rng.choice([0, 7, -13, 123456789])
    if t == "number":
        return rng.choice([0, -1.5, 2.25e10, 3, 1e-7])
    if t == "boolean":
        return rng.random() < 0.5
    if t == "null":
        return None
    if t == "array":
        return [_random_instance(rng, sch["items"])
                for _ in range(rng.randint(sch["minItems"], sch["maxItems"]))]
    req = set(sch.get("required", sch["properties"]))
    return {n: _random_instance(rng, s) for n, s in sch["properties"].items()
            if n in req or rng.random() < 0.5}


def test_random_schemas_accept_their_instances_and_reject_damage():
    import json
    import random
    from arcticinference_b200.structured.json_schema import CompiledSchema
    rng = random.Random(5)
    rejected = damaged = 0
    for _ in range(150):
        sch = _random_schema(rng)
        c = CompiledSchema(sch)
        for _ in range(4):
            doc = _random_instance(rng, sch)
            text = json.dumps(doc, separators=(",", ":"), ensure_ascii=rng.random() < 0.5)
            assert c.validate(text), (sch, text)
            # every proper prefix is a live state, and only whole documents are complete
            st = c.start()
            for ch in text[:-1]:
                st = c.advance(st, ch)
                assert st is not None, (sch, text)
            # damage: drop or double one structural character
            if len(text) > 1:
                i = rng.randrange(len(text))
                bad = text[:i] + text[i + 1:] if rng.random() < 0.5 else text[:i] + text[i] + text[i:]
                try:
                    same = json.loads(bad) == doc
                except ValueError:
                    same = False
                if not same and not c.validate(bad):
                    rejected += 1
                damaged += not same
    assert damaged > 100 and rejected > 0.5 * damaged     # most damaged texts are refused


def _random_regex(rng, depth=0):
    atoms = ["a", "b", "c", r"\d", r"\w", ".", "[ab]", "[^a]", "[a-c0-2]", r"\."]
    def atom():
        if depth < 2 and rng.random() < 0.3:
            return "(" + _random_regex(rng, depth + 1) + ")"
        return rng.choice(atoms)
    parts = []
    for _ in range(rng.randint(1, 4)):
        a = atom()
        q = rng.choice(["", "", "", "?", "*", "+", "{2}", "{1,2}", "{0,3}"])
        parts.append(a + q)
    body = "".join(parts)
    if depth < 2 and rng.random() < 0.3:
        body += "|" + _random_regex(rng, depth + 1)
    return body


def test_random_regexes_agree_with_re_on_random_strings():
    import random
    import re
    from arcticinference_b200.structured.regex import CompiledRegex
    rng = random.Random(11)
    checked = matched = 0
    for _ in range(200):
        pat = _random_regex(rng)
        c = CompiledRegex(pat)
        for _ in range(25):
            s = "".join(rng.choice("abc01. x") for _ in range(rng.randint(0, 7)))
            want = re.fullmatch(pat, s) is not None
            assert c.validate(s) == want, (pat, s, want)
            checked += 1
            matched += want
    assert checked == 5000 and matched > 100
