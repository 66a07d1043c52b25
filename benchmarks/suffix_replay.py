"""Suffix-decoding speculation on the CPU (no GPU, no model): the benchmark configuration
"256 requests of a 512-token prompt and a 256-token response drawn from Zipf(1.1) with n-gram
reuse, global tree over the first 128 responses plus a per-request prompt tree, depth 64, at
most 32 speculated tokens", replayed by ``suffix_replay.cc`` through this package's suffix tree
and, when a copy of the reference is present under ``baseline/_ref``, through the reference's
tree with the very same driver. Prints one JSON line per tree: mean accepted length (tokens per
step including the bonus token) and speculation time per step.

    python benchmarks/suffix_replay.py [--num-requests 256 --train-requests 128 ...]
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from arcticinference_b200.suffix_decoding.simulator import synthetic_requests  # noqa: E402

OURS = os.path.join(ROOT, "arcticinference_b200", "csrc", "suffix_tree")
REFERENCE = os.path.join(ROOT, "baseline", "_ref", "arctic_inference", "csrc", "suffix_decoding")
DRIVER = os.path.join(ROOT, "benchmarks", "suffix_replay.cc")


def build(tmp: str, reference: bool) -> str:
    exe = os.path.join(tmp, "replay_ref" if reference else "replay_ours")
    src_dir = REFERENCE if reference else OURS
    cmd = ["g++", "-O3", "-std=c++20", "-DNDEBUG", "-I", src_dir, DRIVER,
           os.path.join(src_dir, "suffix_tree.cc"), "-o", exe]
    if reference:
        cmd.insert(1, "-DUSE_REFERENCE_TREE")
    subprocess.run(cmd, check=True)
    return exe


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--num-requests", type=int, default=256)
    ap.add_argument("--train-requests", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--response-len", type=int, default=256)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-depth", type=int, default=64)
    ap.add_argument("--max-spec-tokens", type=int, default=32)
    ap.add_argument("--repeat", type=int, default=3, help="runs per tree; the fastest is reported")
    a = ap.parse_args(argv)
    reqs = synthetic_requests(a.num_requests, a.prompt_len, a.response_len, a.vocab, seed=a.seed)
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        trace = os.path.join(tmp, "trace.bin")
        with open(trace, "wb") as f:
            np.asarray([a.num_requests, a.train_requests, a.prompt_len, a.response_len],
                       dtype=np.int32).tofile(f)
            for p, r in reqs:
                np.asarray(p, dtype=np.int32).tofile(f)
                np.asarray(r, dtype=np.int32).tofile(f)
        which = [False] + ([True] if os.path.exists(os.path.join(REFERENCE, "suffix_tree.cc")) else [])
        for reference in which:
            exe = build(tmp, reference)
            best = None
            for _ in range(a.repeat):
                line = subprocess.run([exe, trace, str(a.max_depth), str(a.max_spec_tokens), "1.0",
                                       "0.0", "0.1"], check=True, capture_output=True,
                                      text=True).stdout.strip().splitlines()[-1]
                res = json.loads(line)
                if best is None or res["spec_us_per_step"] < best["spec_us_per_step"]:
                    best = res
            print(json.dumps(best))
            out.append(best)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
