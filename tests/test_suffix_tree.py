"""Suffix tree (C++): structural invariants under random edits, speculation against a
brute-force n-gram oracle, and removal equivalence."""

import random
from collections import Counter

import numpy as np
import pytest

from arcticinference_b200.suffix_decoding import SuffixDecodingCache
from arcticinference_b200.suffix_decoding.cache import SuffixTree


def _rand_seq(rng, n, vocab):
    # repetitive text: random walk over a small set of phrases
    phrases = [[rng.randrange(vocab) for _ in range(rng.randint(2, 6))] for _ in range(6)]
    out = []
    while len(out) < n:
        out += rng.choice(phrases)
        if rng.random() < 0.3:
            out.append(rng.randrange(vocab))
    return out[:n]


def _continuations(seqs, depth, pattern):
    """Counter of next tokens after every occurrence of `pattern` inside a stored string."""
    c = Counter()
    total = 0
    m = len(pattern)
    for s in seqs.values():
        for i in range(len(s) - m + 1):
            if s[i:i + m] == pattern:
                total += 1          # an occurrence at the very end has no continuation
                if i + m < len(s) and m + 1 <= depth:
                    c[s[i + m]] += 1
    return c, total


@pytest.mark.parametrize("depth", [4, 8, 64])
def test_random_edits_keep_invariants(depth):
    rng = random.Random(depth)
    t = SuffixTree(depth)
    live = {}
    for step in range(300):
        op = rng.random()
        if op < 0.5 or not live:
            sid = rng.randrange(40)
            toks = _rand_seq(rng, rng.randint(1, 30), 12)
            t.extend(sid, toks)
            live.setdefault(sid, []).extend(toks)
        elif op < 0.8:
            sid = rng.choice(list(live))
            tok = rng.randrange(12)
            t.append(sid, tok)
            live[sid].append(tok)
        else:
            sid = rng.choice(list(live))
            t.remove(sid)
            del live[sid]
        assert t.check_integrity() == "", "step %d" % step
        assert t.num_seqs() == len(live)
    for sid in list(live):
        t.remove(sid)
        assert t.check_integrity() == ""
    assert t.num_nodes() == 1 and t.num_seqs() == 0


def test_path_speculation_follows_most_frequent_continuation():
    rng = random.Random(1)
    depth = 16
    t = SuffixTree(depth)
    seqs = {i: _rand_seq(rng, 120, 8) for i in range(6)}
    for sid, s in seqs.items():
        t.extend(sid, s)
    assert t.check_integrity() == ""
    checked = 0
    for _ in range(200):
        s = seqs[rng.randrange(6)]
        end = rng.randint(3, len(s) - 1)
        ctx = s[max(0, end - 10):end]
        d = t.speculate(ctx, 8, 4.0, 0.0, 0.0, False)
        assert len(d.token_ids) == len(d.parents) == len(d.probs)
        if not d.token_ids:
            continue
        m = d.match_len
        assert ctx[-m:] == ctx[len(ctx) - m:]
        assert d.parents == list(range(-1, len(d.token_ids) - 1))
        # first token: arg-max of the brute-force continuation counts of the matched suffix
        cont, total = _continuations(seqs, depth, ctx[-m:])
        assert cont, "matched suffix must occur in the data"
        best = max(cont.values())
        assert cont[d.token_ids[0]] == best
        assert abs(d.probs[0] - best / total) < 1e-5
        assert abs(d.score - sum(d.probs)) < 1e-4
        checked += 1
    assert checked > 100


def test_tree_speculation_is_a_tree_ordered_by_probability():
    rng = random.Random(2)
    t = SuffixTree(12)
    seqs = {i: _rand_seq(rng, 150, 6) for i in range(5)}
    for sid, s in seqs.items():
        t.extend(sid, s)
    s = seqs[0]
    d = t.speculate(s[40:48], 12, 4.0, 0.0, 0.05, True)
    assert d.token_ids
    for i, p in enumerate(d.parents):
        assert -1 <= p < i
        if p >= 0:
            assert d.probs[i] <= d.probs[p] + 1e-6
    assert all(pr >= 0.05 - 1e-6 for pr in d.probs)
    # best-first: probabilities are emitted in non-increasing order
    assert all(d.probs[i] >= d.probs[i + 1] - 1e-6 for i in range(len(d.probs) - 1))


def test_remove_equals_never_added():
    rng = random.Random(3)
    a, b = SuffixTree(10), SuffixTree(10)
    seqs = {i: _rand_seq(rng, 80, 7) for i in range(8)}
    for sid, s in seqs.items():
        a.extend(sid, s)
    for sid in (1, 4, 6):
        a.remove(sid)
    for sid, s in seqs.items():
        if sid not in (1, 4, 6):
            b.extend(sid, s)
    assert a.check_integrity() == "" and b.check_integrity() == ""
    assert a.num_nodes() == b.num_nodes()
    for _ in range(300):
        s = seqs[rng.choice([0, 2, 3, 5, 7])]
        end = rng.randint(2, len(s))
        ctx = s[max(0, end - 8):end]
        # one-token drafts are independent of how ties between equally frequent siblings
        # happen to be ordered, which depends on the insertion history
        da, db = a.speculate(ctx, 1, 2.0, 0.0, 0.0, False), b.speculate(ctx, 1, 2.0, 0.0, 0.0, False)
        assert da.match_len == db.match_len and len(da.token_ids) == len(db.token_ids)
        assert np.allclose(da.probs, db.probs, atol=1e-6)


def test_budget_rules():
    t = SuffixTree(64)
    t.extend(0, list(range(100)))
    d = t.speculate([5, 6, 7], 32, 1.0, 0.0, 0.1, False)
    assert d.match_len == 3 and d.token_ids == [8, 9, 10]          # floor(3 * 1.0 + 0)
    d = t.speculate([5, 6, 7], 32, 2.0, 1.0, 0.1, False)
    assert d.token_ids == list(range(8, 15))                        # floor(3 * 2 + 1) = 7
    d = t.speculate([5, 6, 7], 2, 2.0, 1.0, 0.1, False)
    assert d.token_ids == [8, 9]
    assert t.speculate([200, 201], 8, 1.0, 0.0, 0.1, False).token_ids == []


def test_cache_lifecycle_and_eviction():
    c = SuffixDecodingCache(max_tree_depth=16, max_cached_requests=2)
    prompt = list(range(10, 40))
    c.start_request("a", prompt)
    c.add_active_response("a", [40, 41, 42, 10, 11, 12])
    d = c.speculate("a", [10, 11, 12], max_spec_tokens=4)
    assert d.token_ids[:3] == [13, 14, 15]          # copied from the prompt (local tree)
    c.stop_request("a")
    c.start_request("b", [1, 2, 3])
    d = c.speculate("b", [40, 41], max_spec_tokens=3, max_spec_factor=2.0)
    assert d.token_ids[:1] == [42]                  # from a's cached response (global tree)
    c.add_active_response("b", [7, 7, 7])
    c.stop_request("b")
    c.start_request("c", [5])
    c.stop_request("c")
    assert c.num_cached_requests == 2 and "a" not in c.cached_requests   # FIFO eviction
    assert c.check_integrity() == ""
    with pytest.raises(ValueError):
        c.speculate("zzz", [1, 2])
    assert c.max_depth == 16


def test_fuzz_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The C++ tree alone (no interpreter in the process), compiled with ASAN + UBSAN, under
    random append / remove / speculate traffic with an integrity check after every operation."""
    import os
    import shutil
    import subprocess
    # the first compiler that links against the sanitizer runtimes (a toolchain installed
    # beside the system one often lacks them)
    cands = [c for c in (os.environ.get("CXX"), "/usr/bin/g++", shutil.which("g++"),
                         shutil.which("clang++")) if c and os.path.exists(c)]
    if not cands:
        pytest.skip("no C++ compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "arcticinference_b200", "csrc", "suffix_tree")
    exe = str(tmp_path / "suffix_fuzz")
    for cxx in cands:
        build = subprocess.run(
            [cxx, "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined",
             "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-I", src,
             os.path.join(root, "tests", "suffix_tree_fuzz.cc"),
             os.path.join(src, "suffix_tree.cc"), "-o", exe], capture_output=True, text=True)
        if build.returncode == 0:
            break
    if build.returncode != 0 and "cannot find" in build.stderr and "san" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    for seed in (1, 2, 3):
        run = subprocess.run([exe, str(seed), "400"], capture_output=True, text=True, timeout=300,
                             env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1"))
        assert run.returncode == 0 and run.stdout.strip() == "ok", (run.stdout + run.stderr)[-3000:]
